"""-m gpu: the profiling aids of the session (step timeline, per-CTA GEMM trace, timing-only ablation)
and the multi-block arg-max, through the C ABI. They must report sane values and must leave the
session's results untouched once they are switched off."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _session(model_dirs, name="mini05", n=4, max_seq=128):
    import synth
    import tffn
    d, ep, cfg = model_dirs[name]
    m = tffn.qwen_load(d)
    e = tffn.checkpoint_load(ep, m, 0.1)
    s = tffn.Session(m, e, max_batch=n, max_seq=max_seq)
    prompts = [synth.prompts(1, 9 + 3 * i, 300 + i, cfg["vocab_size"])[0] for i in range(n)]
    return m, e, s, prompts, cfg


@pytest.mark.parametrize("mode", [1, 2])
def test_timeline_reports_every_launch_in_order(model_dirs, mode):
    m, e, s, prompts, cfg = _session(model_dirs)
    s.set_launch_mode(mode)
    s.prefill(prompts)
    before = [s.seq_len(i) for i in range(4)]
    names, tl, tr = s.timeline(4, trace_launch=2, trace_ctas=4096)  # launch 2 = the first q|k|v GEMM
    L = cfg["num_hidden_layers"]
    assert len(names) == 1 + 7 * L + 3  # embed, 7 per layer, final norm, LM head, arg-max
    assert names[0] == "embed_rows" and names[2] == "gemm_tc:qkv" and names[-1] == "argmax_rows"
    assert names.count("attn_decode") == L and names.count("gemm_tc:down") == L
    t = tl.astype(np.int64)
    assert (t > 0).all()
    assert (t[:, 0] <= t[:, 1]).all() and (t[:, 2] <= t[:, 3]).all() and (t[:, 4] <= t[:, 5]).all()
    assert (t[:, 0] <= t[:, 5]).all()
    # a kernel leaves its grid wait only after the previous kernel of the stream has finished
    assert (t[1:, 2] >= t[:-1, 5]).all()
    span_us = (t[:, 5].max() - t[:, 0].min()) / 1e3
    assert 1.0 < span_us < 1e5
    # per-CTA phase stamps of the traced GEMM: start <= dependency wait over <= end, inside the launch
    live = tr[:, 0] > 0
    assert live.sum() >= 1
    c = tr[live].astype(np.int64)
    assert (c[:, 0] <= c[:, 8]).all() and (c[:, 8] <= t[2, 5] + 1000).all()
    # the three diagnostic steps advanced the sequences like ordinary decode steps
    assert [s.seq_len(i) for i in range(4)] == [b + 3 for b in before]
    assert s.status() == 0


def test_ablation_is_timing_only_and_restores(model_dirs):
    m, e, s, prompts, cfg = _session(model_dirs)
    s.set_launch_mode(2)
    s.prefill(prompts)
    ref = s.decode_run(4, 6)
    s.qwen_reset()
    s.prefill(prompts)
    s.set_ablation(1 << 3)  # skip the attention kernel: results are garbage but the step must run
    s.decode_run(4, 2, want_tokens=False)
    assert s.status() == 0
    s.set_ablation(0)
    s.qwen_reset()
    s.prefill(prompts)
    again = s.decode_run(4, 6)
    assert (ref == again).all()


def test_argmax_many_blocks_first_maximum(model_dirs):
    """greedy picks of a batched step == numpy argmax (first index among equal maxima) of its logits"""
    m, e, s, prompts, cfg = _session(model_dirs, "mini05", n=4)
    nxt, lg = s.prefill(prompts, want_logits=True)
    assert (np.asarray(nxt) == lg.argmax(-1)).all()
    for _ in range(3):
        nxt, lg = s.decode_step(nxt, want_logits=True)
        assert (np.asarray(nxt) == lg.argmax(-1)).all()
