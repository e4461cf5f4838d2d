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
                                   (100, 640, 256), (200, 448, 608), (300, 896, 4864), (513, 256, 64),
                                   # few wide tiles, short K: split 8 ways into clusters whose rings are then cut back so
                                   # that all of them are resident at once (the parked plane must still fit the ring)
                                   (512, 896, 896), (256, 1152, 896), (130, 896, 896), (32, 2304, 3584)])
def test_gemm_matches_numpy(T, N, K):
    import tffn
    rng = np.random.default_rng([T, N, K])
    X, W = _rand_bf16(rng, (T, K)), _rand_bf16(rng, (N, K), 0.05)
    out = tffn.op_gemm(X, W)
    ref = _ref(X, W)
    err = np.abs(out - ref).max() / np.abs(ref).max()
    assert err < 2e-5, err  # fp32 accumulation of exact bf16 products


@pytest.mark.parametrize("splits", [1, 2, 4, 8, 16])
def test_gemm_split_k_is_deterministic(splits):
    import tffn
    rng = np.random.default_rng(99)
    X, W = _rand_bf16(rng, (48, 1024)), _rand_bf16(rng, (256, 1024), 0.05)
    a = tffn.op_gemm(X, W, splits=splits)
    b = tffn.op_gemm(X, W, splits=splits)
    assert (a == b).all()
    ref = _ref(X, W)
    assert np.abs(a - ref).max() / np.abs(ref).max() < 2e-5


def _ffn_ref(h, w, gate, up, down, eps):
    """numpy restatement of one FFN branch input/outputs in float64 with the bf16 rounding points of
    inference/src/model/qwen.cu:422-437 (rmsnorm -> bf16, gate/up -> bf16, act -> bf16, down fp32)"""
    import synth
    f, r = synth.bf16_to_f32, lambda x: synth.bf16_to_f32(synth.f32_to_bf16(np.asarray(x, dtype=np.float32)))
    x = f(h).astype(np.float64)
    xn = r(x * (1.0 / np.sqrt((x * x).mean() + eps)) * f(w))
    g, u = r(f(gate).astype(np.float64) @ xn), r(f(up).astype(np.float64) @ xn)
    act = r((g / (1.0 + np.exp(-g.astype(np.float64)))) * u)
    return f(down).astype(np.float64) @ act


@pytest.mark.parametrize("H,I,expert", [(256, 96, True), (896, 4864, True), (896, 4864, False), (448, 1216, True),
                                        (1536, 8960, True), (2048, 2752, True)])
def test_fused_bs1_ffn_kernel(H, I, expert):
    """the fused batch-1 SwiGLU kernel alone, at sizes where every CTA's ring wraps several times"""
    import synth
    import tffn
    rng = np.random.default_rng([H, I])
    h = _rand_bf16(rng, (H,))
    w = synth.f32_to_bf16(1.0 + 0.1 * rng.standard_normal(H, dtype=np.float32))
    mats = [[_rand_bf16(rng, s, 0.02) for s in ((I, H), (I, H), (H, I))] for _ in range(2)]
    pb, pe = tffn.pack_ffn(*mats[0]), tffn.pack_ffn(*mats[1])
    out = synth.bf16_to_f32(tffn.op_swiglu_bs1(h, w, pb, pe if expert else None, 0.1, 1e-6))
    ref = synth.bf16_to_f32(h).astype(np.float64) + _ffn_ref(h, w, *mats[0], 1e-6)
    if expert:
        ref = ref + 0.1 * _ffn_ref(h, w, *mats[1], 1e-6)
    scale = np.abs(ref).max()
    assert np.abs(out - ref).max() / scale <= 1e-2   # one bf16 ulp of the largest element is 0.8 %
    assert np.abs(out - ref).mean() / scale <= 1.5e-3
    again = synth.bf16_to_f32(tffn.op_swiglu_bs1(h, w, pb, pe if expert else None, 0.1, 1e-6))
    assert (again == out).all()  # fixed reduction order
