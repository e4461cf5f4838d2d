"""-m gpu, needs at least two GPUs (skipped otherwise): tensor-parallel ranks, one process per GPU, against the
same model on one GPU. Every rank must return the same tokens and the same full logits, within the kernel
tolerance of the single-GPU result (the fp32 sum over the ranks changes the order of summation, nothing else),
through both exchange paths: partial sums pushed into the peers' windows (decode-sized launches) and NCCL.
Failure handling is covered without any GPU fault by tests/test_tp_cpu.py (a rank that never arrives)."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KERNEL_TOL = 1.5e-2

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    sys.path.insert(0, os.path.join(%r, "tensor-ffn_b200"))
    import synth, tffn
    rank, size, meet, d, ep, out, mode = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3], sys.argv[4], sys.argv[5], sys.argv[6], int(sys.argv[7])
    fused = int(sys.argv[8])
    g = None
    if size > 1:
        g = tffn.TpGroup(tffn.tp_rendezvous(meet, rank, size, 120.0), rank, size, rank)
    m = tffn.qwen_load(d, device=rank, tp_rank=rank, tp_size=size)
    e = tffn.checkpoint_load(ep, m, 0.1)
    V = m.cfg.vocab_size
    s = tffn.Session(m, e, max_batch=3, max_seq=96, tp=g)
    s.set_launch_mode(mode)
    if size > 1:
        s.set_tp_fused(bool(fused))
    prompts = [synth.prompts(1, n, 500 + i, V)[0] for i, n in enumerate((9, 17, 5))]
    forced = synth.prompts(3, 5, 600, V)
    nxt, lg = s.prefill(prompts, want_logits=True)
    rows = [lg.copy()]
    for k in range(5):
        nxt, lg = s.decode_step(forced[:, k], want_logits=True)
        rows.append(lg.copy())
    toks = s.decode_run(3, 6)
    one = s.qwen_forward(synth.prompts(1, 11, 700, V)[0], slot=0) if False else None
    assert s.status() == 0
    np.savez(out, logits=np.array(rows), tokens=np.asarray(toks), last=np.asarray(nxt))
    s.free(); e.free(); m.free()
    if g: g.free()
""")


def _run(tmp_path, d, ep, size, mode, tag, fused=1):
    script = tmp_path / "tp_worker.py"
    script.write_text(WORKER % ROOT)
    meet = tmp_path / f"meet_{tag}"
    procs = []
    for r in range(size):
        out = tmp_path / f"out_{tag}_{r}.npz"
        procs.append((subprocess.Popen([sys.executable, str(script), str(r), str(size), str(meet), d, ep, str(out), str(mode), str(fused)],
                                       stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                                       env=dict(os.environ, NCCL_NVLS_ENABLE="0")), out))
    res = []
    for p, out in procs:
        try:
            log, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            raise AssertionError("tensor-parallel worker did not finish")
        assert p.returncode == 0, log[-3000:]
        res.append(np.load(out))
    return res


@pytest.mark.parametrize("mode", [1, 2])
def test_two_ranks_match_one_gpu(model_dirs, tmp_path, mode):
    import tffn
    if tffn.device_count() < 2:
        pytest.skip("needs two GPUs")
    d, ep, cfg = model_dirs["tiny"]  # 4 query / 2 kv heads, intermediate 512, vocabulary 1024: splits in two
    one = _run(tmp_path, d, ep, 1, mode, f"tp1_{mode}")[0]
    two = _run(tmp_path, d, ep, 2, mode, f"tp2_{mode}")  # decode-sized launches over peer memory
    nccl = _run(tmp_path, d, ep, 2, mode, f"tp2n_{mode}", fused=0)  # every all-reduce through NCCL
    # both ranks: identical results (they hold the same sums, added in the same order, and the same exchanged
    # candidates)
    for res in (two, nccl):
        assert (res[0]["logits"] == res[1]["logits"]).all() and (res[0]["tokens"] == res[1]["tokens"]).all()
    # the two exchange paths add the same two fp32 partial sums (a + b = b + a) and share the row arithmetic
    assert (two[0]["logits"] == nccl[0]["logits"]).all() and (two[0]["tokens"] == nccl[0]["tokens"]).all()
    a, b = two[0]["logits"], one["logits"]
    assert np.isfinite(a).all()
    assert np.abs(a - b).max() / np.abs(b).max() <= KERNEL_TOL
    # picks: equal wherever the single-GPU logits are not nearly tied
    pa, pb = a.argmax(-1), b.argmax(-1)
    err = np.abs(a - b).max()
    gap = np.take_along_axis(b, pb[..., None], -1)[..., 0] - np.take_along_axis(b, pa[..., None], -1)[..., 0]
    assert ((pa == pb) | (gap <= 2 * err)).all()


@pytest.mark.parametrize("size", [4, 8])
def test_wider_groups_split_a_kv_head(model_dirs, tmp_path, size):
    """4 and 8 ranks on the 7B head geometry (14 query / 2 kv heads): two or four ranks share a kv head and
    split its seven query heads 3 + 4 or 1 + 2 + 2 + 2. All ranks identical, within tolerance of one GPU,
    through both exchange paths."""
    import tffn
    if tffn.device_count() < size:
        pytest.skip(f"needs {size} GPUs")
    d, ep, cfg = model_dirs["mini7"]
    one = _run(tmp_path, d, ep, 1, 2, "w_tp1")[0]
    for fused in (1, 0):
        res = _run(tmp_path, d, ep, size, 2, f"w_tp{size}_{fused}", fused=fused)
        for r in res[1:]:
            assert (res[0]["logits"] == r["logits"]).all() and (res[0]["tokens"] == r["tokens"]).all()
        a, b = res[0]["logits"], one["logits"]
        assert np.isfinite(a).all()
        assert np.abs(a - b).max() / np.abs(b).max() <= KERNEL_TOL, (size, fused)
