"""-m gpu: the tcgen05 GEMM of the batched path alone, against numpy on the same bf16 inputs."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _rand_bf16(rng, shape, scale=1.0):
    import synth
    return synth.f32_to_bf16((rng.standard_normal(shape, dtype=np.float32) * scale).reshape(-1)).reshape(shape)


def _ref(X, W):
    import synth
    return synth.bf16_to_f32(X).astype(np.float64) @ synth.bf16_to_f32(W).astype(np.float64).T


@pytest.mark.parametrize("T,N,K", [(1, 128, 64), (5, 256, 128), (16, 384, 448), (17, 1000, 896), (64, 1152, 896),
                                   (100, 640, 256), (200, 448, 608), (300, 896, 4864), (513, 256, 64)])
def test_gemm_matches_numpy(T, N, K):
    import tffn
    rng = np.random.default_rng([T, N, K])
    X, W = _rand_bf16(rng, (T, K)), _rand_bf16(rng, (N, K), 0.05)
    out = tffn.op_gemm(X, W)
    ref = _ref(X, W)
    err = np.abs(out - ref).max() / np.abs(ref).max()
    assert err < 2e-5, err  # fp32 accumulation of exact bf16 products


@pytest.mark.parametrize("splits", [1, 2, 3, 7])
def test_gemm_split_k_is_deterministic(splits):
    import tffn
    rng = np.random.default_rng(99)
    X, W = _rand_bf16(rng, (48, 1024)), _rand_bf16(rng, (256, 1024), 0.05)
    a = tffn.op_gemm(X, W, splits=splits)
    b = tffn.op_gemm(X, W, splits=splits)
    assert (a == b).all()
    ref = _ref(X, W)
    assert np.abs(a - ref).max() / np.abs(ref).max() < 2e-5
