"""CPU: host logic of tensor parallelism (BASELINE.json configs[4]: the 7B shape split over 2 / 4 / 8 GPUs) —
the partition arithmetic (every head, every intermediate row, every LM-head row owned exactly once; the
uneven 3 + 4 split of a kv group's query heads at TP 8), a world-size-2 gloo run in which the ranks
exchange what they own, and the meeting point that gives up when a rank never arrives. No GPU, no NCCL."""
import os
import socket
import subprocess
import sys
import textwrap
import threading

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _cfg(tffn, H, I, L, nh, nkv, V):
    c = tffn.Config()
    c.hidden_size, c.intermediate_size, c.num_layers, c.num_heads, c.num_kv_heads = H, I, L, nh, nkv
    c.head_dim, c.vocab_size = H // nh, V
    return c


@pytest.mark.parametrize("tp", [1, 2, 4, 8])
def test_partition_of_the_7b_shape_covers_everything_once(tp):
    import tffn
    c = _cfg(tffn, 3584, 18944, 28, 28, 4, 152064)
    parts = [tffn.tp_partition(c, r, tp) for r in range(tp)]
    q = sorted(h for p in parts for h in range(p["q_head0"], p["q_head0"] + p["n_q_heads"]))
    assert q == list(range(28))                                             # every query head exactly once
    rows = sorted(i for p in parts for i in range(p["i0"], p["i0"] + p["n_i"], 64))
    assert rows == list(range(0, 18944, 64)) and all(p["n_i"] % 64 == 0 for p in parts)
    v = sorted(i for p in parts for i in range(p["v0"], p["v0"] + p["n_v"], 8))
    assert v == list(range(0, 152064, 8)) and len({p["n_v"] for p in parts}) == 1   # even split: logits can be gathered
    for p in parts:
        # a rank's query heads all belong to the kv heads it holds (GQA map kv = q * nkv / nh, qwen.cu:252)
        kv_of_q = {h * 4 // 28 for h in range(p["q_head0"], p["q_head0"] + p["n_q_heads"])}
        assert kv_of_q <= set(range(p["kv_head0"], p["kv_head0"] + p["n_kv_heads"]))
        assert p["n_q_heads"] % p["n_kv_heads"] == 0 and p["n_q_heads"] // p["n_kv_heads"] <= 8
    if tp <= 4:
        assert sorted(k for p in parts for k in range(p["kv_head0"], p["kv_head0"] + p["n_kv_heads"])) == list(range(4))
    else:  # two ranks share each kv head and split its 7 query heads 3 + 4
        assert [p["n_q_heads"] for p in parts] == [3, 4] * 4
        assert [p["kv_head0"] for p in parts] == [0, 0, 1, 1, 2, 2, 3, 3]


def test_partition_rejects_what_does_not_split():
    import tffn
    c = _cfg(tffn, 896, 4864, 24, 14, 2, 151936)
    assert tffn.tp_partition(c, 1, 2)["n_q_heads"] == 7
    with pytest.raises(tffn.TffnError):
        tffn.tp_partition(c, 0, 3)        # 2 kv heads over 3 ranks
    with pytest.raises(tffn.TffnError):
        tffn.tp_partition(c, 2, 2)        # rank out of range
    c2 = _cfg(tffn, 256, 200, 2, 4, 2, 1024)
    with pytest.raises(tffn.TffnError):
        tffn.tp_partition(c2, 0, 2)       # intermediate size not a multiple of 64


WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, os.path.join(%r, "tensor-ffn_b200"))
    import torch.distributed as dist
    import tffn
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    c = tffn.Config()
    c.hidden_size, c.intermediate_size, c.num_layers, c.num_heads, c.num_kv_heads, c.head_dim, c.vocab_size = 3584, 18944, 28, 28, 4, 128, 152064
    mine = tffn.tp_partition(c, rank, world)
    everyone = [None] * world
    dist.all_gather_object(everyone, mine)
    assert everyone[rank] == mine
    assert sum(p["n_q_heads"] for p in everyone) == 28 and sum(p["n_i"] for p in everyone) == 18944
    assert sum(p["n_v"] for p in everyone) == 152064
    # the id travels from rank 0 to the others as 128 opaque bytes (here a stand-in: no NCCL on this machine)
    box = [bytes(range(128)) if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    assert len(box[0]) == 128
    dist.barrier()
    if rank == 0:
        print("tp host logic ok", world)
    dist.destroy_process_group()
""")


def test_two_ranks_exchange_their_partitions_over_gloo(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), str(script)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "tp host logic ok 2" in r.stdout


def test_rendezvous_gives_up_when_a_rank_never_arrives(tmp_path, monkeypatch):
    """rank 1 of 2 never shows up: rank 0 gets a status code after the timeout instead of hanging in a collective"""
    import tffn
    monkeypatch.setattr(tffn, "tp_unique_id", lambda: bytes(128))  # no NCCL here; the id's content is irrelevant
    with pytest.raises(tffn.TffnError) as ei:
        tffn.tp_rendezvous(str(tmp_path / "a"), 0, 2, timeout_s=0.3)
    assert ei.value.code == -6 and "[1]" in ei.value.msg
    # and when both arrive, both get the id
    got = {}
    th = threading.Thread(target=lambda: got.setdefault(1, tffn.tp_rendezvous(str(tmp_path / "b"), 1, 2, timeout_s=10)))
    th.start()
    got[0] = tffn.tp_rendezvous(str(tmp_path / "b"), 0, 2, timeout_s=10)
    th.join()
    assert got[0] == got[1] == bytes(128)
