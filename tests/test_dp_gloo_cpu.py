"""CPU, world_size 2 over gloo: the host logic of the multi-GPU (data-parallel) bench — sharding of
sequences over ranks with nothing shared, rank-0-only model generation behind a barrier, and the
max-over-ranks reduction of the timed region. No collective exists on the data path itself."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, %r); sys.path.insert(0, os.path.join(%r, "tensor-ffn_b200"))
    import numpy as np, torch, torch.distributed as dist
    import bench
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    n, plen = 4, 16
    ids = bench.dp_sequence_ids(rank, n)
    p = bench.dp_prompts(rank, n, plen)
    gathered = [None] * world
    dist.all_gather_object(gathered, (ids, p.tolist()))
    all_ids = sum((g[0] for g in gathered), [])
    assert sorted(all_ids) == list(range(world * n)), all_ids          # a partition of the global sequences
    rows = {tuple(r) for g in gathered for r in g[1]}
    assert len(rows) == world * n                                        # distinct prompts everywhere
    import synth
    assert (p == synth.prompts(world * n, plen, 1)[rank * n:(rank + 1) * n]).all()  # same as the unsharded job
    # rank 0 prepares shared state, the others wait at the barrier before reading it
    marker = os.path.join(os.environ["TFFN_TMP"], "ready")
    if rank == 0:
        open(marker, "w").write("ok")
    dist.barrier()
    assert os.path.exists(marker)
    t = bench.reduce_max(dist, 10.0 + rank, "cpu")
    assert t == 10.0 + world - 1
    value = world * n * 8 / (t / 1e3)                                    # whole-job throughput from the slowest rank
    if rank == 0:
        print(json.dumps({"value": value, "ranks": world}))
    dist.barrier()
    dist.destroy_process_group()
""")


def test_two_rank_data_parallel_host_logic(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % (ROOT, ROOT))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, TFFN_TMP=str(tmp_path))
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
                        "127.0.0.1", "--master-port", str(port), str(script)], capture_output=True, text=True, env=env,
                       timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert '"ranks": 2' in r.stdout
