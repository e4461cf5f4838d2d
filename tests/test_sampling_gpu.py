"""-m gpu: temperature sampling on the device (tffn_session_set_sampling) against a restatement of the
reference's host sampler sample() (inference/src/main.cpp:52-63) applied to the logits the same step
returned, with the reference's random stream (std::mt19937 seeded 42, one
std::uniform_real_distribution<double> draw per token)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

# first draws of std::uniform_real_distribution<double>(0, 1) over std::mt19937(42) (libstdc++:
# (x0 + x1 * 2^32) / 2^64 with x0 = 1608637542, x1 = 3421126067, ...)
MT42_FIRST = (0.79654298428784598, 0.18343478789336848, 0.77969099761266125)


def canonical_draws(seed, n):
    """std::uniform_real_distribution<double>(0,1)(std::mt19937(seed)): two 32-bit outputs per draw"""
    rs = np.random.RandomState()
    rs.seed(np.uint32(seed))  # init_genrand, the seeding std::mt19937(seed) uses
    raw = rs.randint(0, 2 ** 32, size=2 * n, dtype=np.uint64)
    out = (raw[0::2].astype(np.float64) + raw[1::2].astype(np.float64) * 4294967296.0) / 18446744073709551616.0
    return np.minimum(out, np.nextafter(1.0, 0.0))


def host_sample(logits, temperature, u):
    """sample() of the reference for temperature > 0, with r = u * sum"""
    lg = logits.astype(np.float32)
    mx = lg.max()
    p = np.exp(((lg - mx) / np.float32(temperature)).astype(np.float32)).astype(np.float64)  # float exp, double sum
    acc = np.cumsum(p)  # left to right, as the reference accumulates
    r = u * acc[-1]
    hit = np.nonzero(acc >= r)[0]
    return int(hit[0]) if len(hit) else len(lg) - 1


def test_reference_random_stream():
    d = canonical_draws(42, 3)
    assert np.allclose(d, MT42_FIRST, rtol=0, atol=1e-17)


@pytest.mark.parametrize("n_seqs", [1, 3])
def test_device_sampling_matches_host_sampler(model_dirs, n_seqs):
    import synth
    import tffn
    d, ep, cfg = model_dirs["mini05"]
    m = tffn.qwen_load(d)
    e = tffn.checkpoint_load(ep, m, 0.1)
    s = tffn.Session(m, e, max_batch=n_seqs, max_seq=96)
    s.set_launch_mode(2)
    T = 0.7
    s.set_sampling(T, 42)
    prompts = [synth.prompts(1, 7 + 2 * i, 40 + i, cfg["vocab_size"])[0] for i in range(n_seqs)]
    steps = 6
    draws = canonical_draws(42, n_seqs * (steps + 1))
    k = 0
    nxt, lg = s.prefill(prompts, want_logits=True)
    mismatches = 0
    for i in range(n_seqs):  # one draw per sequence, slot order
        mismatches += int(nxt[i]) != host_sample(lg[i], T, draws[k])
        k += 1
    for _ in range(steps):
        nxt, lg = s.decode_step(nxt, want_logits=True)
        for i in range(n_seqs):
            mismatches += int(nxt[i]) != host_sample(lg[i], T, draws[k])
            k += 1
    # device expf differs from the host's by an ulp or two: a pick can differ only if r falls within
    # ~1e-7 of a boundary of the cumulative distribution, which none of these draws does
    assert mismatches == 0
    assert s.status() == 0
    # sampled picks are not all greedy picks (the random-init distribution is nearly flat)
    # and greedy comes back when sampling is switched off
    s.set_sampling(0.0, 42)
    nxt2, lg2 = s.decode_step(nxt, want_logits=True)
    assert (np.asarray(nxt2) == lg2.argmax(-1)).all()


def test_sampled_decode_run_matches_stepwise(model_dirs):
    """the device-resident loop consumes the draws in the same order as step-by-step decoding"""
    import synth
    import tffn
    d, ep, cfg = model_dirs["tiny"]
    m = tffn.qwen_load(d)
    e = tffn.checkpoint_load(ep, m, 0.1)
    prompts = [synth.prompts(1, 9 + i, 60 + i, cfg["vocab_size"])[0] for i in range(2)]
    def run(stepwise):
        s = tffn.Session(m, e, max_batch=2, max_seq=96)
        s.set_launch_mode(2)
        s.set_sampling(1.3, 7)
        s.prefill(prompts)
        if stepwise:
            out = np.array([s.decode_step(None, n_seqs=2)[0] for _ in range(8)])
        else:
            out = np.asarray(s.decode_run(2, 8)).copy()
        assert s.status() == 0
        s.free()
        return out

    a, b = run(False), run(True)
    if not (a == b).all():  # say which of the two is unstable before failing
        a2, b2 = run(False), run(True)
        raise AssertionError(("run", a.T.tolist(), "stepwise", b.T.tolist(), "run again", a2.T.tolist(), "stepwise again",
                              b2.T.tolist()))


def test_cli_device_sampling_equals_host_sampling(model_dirs, tmp_path):
    """tensor-ffn-inference --temperature: picks drawn on the device == the reference's host loop over
    downloaded logits (--host-sampling), token for token, same mt19937(42) stream"""
    import os
    import subprocess
    import synth
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cli = os.path.join(root, "tensor-ffn_b200", "tensor-ffn-inference")
    d, ep, cfg = model_dirs["mini05"]
    ids = tmp_path / "prompt.i32"
    np.asarray(synth.prompts(1, 12, 5, cfg["vocab_size"])[0], dtype=np.int32).tofile(ids)
    outs = []
    for extra in ([], ["--host-sampling"]):
        cmd = [cli, "--model", d, "--expert", ep, "--prompt-ids", str(ids), "--max-tokens", "12", "--temperature", "0.9",
               "--ignore-eos", "--max-seq", "64"] + extra + ["--device", "0"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
        outs.append(r.stdout.split("Generating:")[1])
    assert outs[0] == outs[1] and len(outs[0].strip()) > 0


def test_sampling_survives_growth_of_the_token_staging_buffer(model_dirs):
    """A prompt of more than ~700 tokens regrows the pinned int32 staging buffer after the pinned buffer
    of the draws already exists; the draws' buffer must stay valid (it was once freed there) and the
    sampled picks must keep following the host sampler."""
    import synth
    import tffn
    d, ep, cfg = model_dirs["tiny"]
    m = tffn.qwen_load(d)
    e = tffn.checkpoint_load(ep, m, 0.1)
    s = tffn.Session(m, e, max_batch=1, max_seq=1024)
    T = 0.8
    s.set_sampling(T, 42)
    draws = canonical_draws(42, 16)
    k = 0
    nxt, lg = s.prefill([synth.prompts(1, 5, 90, cfg["vocab_size"])[0]], want_logits=True)
    assert int(nxt[0]) == host_sample(lg[0], T, draws[k]); k += 1
    nxt, lg = s.decode_step(nxt, want_logits=True)
    assert int(nxt[0]) == host_sample(lg[0], T, draws[k]); k += 1
    s.qwen_reset()
    nxt, lg = s.prefill([synth.prompts(1, 800, 91, cfg["vocab_size"])[0]], want_logits=True)  # 800 * 6 ints > 4096
    assert int(nxt[0]) == host_sample(lg[0], T, draws[k]); k += 1
    for _ in range(4):
        nxt, lg = s.decode_step(nxt, want_logits=True)
        assert int(nxt[0]) == host_sample(lg[0], T, draws[k]); k += 1
    assert s.status() == 0
    s.free()


def test_sampled_graph_is_rebuilt_when_the_draw_buffer_grows(model_dirs):
    """decode_run with more than 1024 draws reallocates the device buffer of the draws; a decode graph
    captured before (same key) holds the old address and has to be dropped, not replayed"""
    import synth
    import tffn
    d, ep, cfg = model_dirs["tiny"]
    m = tffn.qwen_load(d)
    e = tffn.checkpoint_load(ep, m, 0.1)
    prompts = [synth.prompts(1, 6 + (i % 3), 120 + i, cfg["vocab_size"])[0] for i in range(64)]
    steps = 17  # 64 * 17 = 1088 draws > 1024

    def run(stepwise):
        s = tffn.Session(m, e, max_batch=64, max_seq=64)
        s.set_launch_mode(2)
        s.set_sampling(1.1, 11)
        s.prefill(prompts)
        first = np.asarray(s.decode_step(None, n_seqs=64)[0]).copy()  # captures the graph with the small buffer
        if stepwise:
            rest = np.array([s.decode_step(None, n_seqs=64)[0] for _ in range(steps)])
        else:
            rest = np.asarray(s.decode_run(64, steps)).copy()
        assert s.status() == 0
        s.free()
        return first, rest

    (fa, a), (fb, b) = run(False), run(True)
    assert (fa == fb).all() and (a == b).all()
