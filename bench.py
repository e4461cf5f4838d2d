#!/usr/bin/env python
"""Decode throughput of the Qwen2.5 + expert-FFN inference path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...  # the reference's own code

Workload (BASELINE.json configs[1]): Qwen2.5-0.5B shape + expert, bf16, 64 independent
sequences per GPU, 512-token uniform-random prompts, greedy decode. A "step" is one decode step
of the whole batch (64 new tokens per GPU). With N > 1 the sequences are sharded data-parallel,
64 per rank, no collective on the data path (weak scaling; a strong-scaling run of 64 sequences
in total rides along as an extra). --tp N (configs[4], the 7B shape) makes the N ranks one
tensor-parallel group instead. Weights are seeded synthetic stand-ins with the real shapes,
written to disk in the reference's file formats and loaded through the library's loader. One
JSON line is printed by rank 0. The timed region of K steps is repeated and the median taken.

value      decode tok/s with everything resident in HBM (device-side loop, CUDA events)
e2e        the same metric through the public C ABI with host buffers: every step copies the
           step's input tokens host->device and the picks device->host
bs1        BASELINE.json configs[0] (batch 1, 128-token prompt) on the same model, as extras
roofline   dominant kernel: algorithmic bytes / its measured device time vs measured HBM peak
"""
from __future__ import annotations

import argparse
import json
import os
import shutil
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(ROOT, "tensor-ffn_b200"))

FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only without MEASURED_PEAKS.json


def metric_name(a) -> str:
    name = {"0.5b": "Qwen2.5-0.5B", "1.5b": "Qwen2.5-1.5B", "3b": "Qwen2.5-3B", "7b": "Qwen2.5-7B"}.get(a.shape, a.shape)
    return f"decode tok/s, {name}+expert bf16 bs{a.seqs} (bs1 in extras); % of HBM roofline"


def workload_name(a) -> str:
    idx = {"0.5b": 1, "1.5b": 2, "3b": 3, "7b": 4}.get(a.shape)
    name = {"0.5b": "Qwen2.5-0.5B", "1.5b": "Qwen2.5-1.5B", "3b": "Qwen2.5-3B", "7b": "Qwen2.5-7B"}.get(a.shape, a.shape)
    tag = f"configs[{idx}] shape" if idx is not None else "custom shape"
    return f"{tag}: {name}+expert, {a.seqs} sequences x {a.prompt}-token prompts, batched greedy decode"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


# DRAM traffic of k_gemm_tc from an ncu capture of two launches
# (one launch each of the two largest decode shapes, 64 tokens): dram read+write bytes per byte of
# weights for a layer-sized launch whose output stays in L2, and the part of the LM head's fp32 logits
# that reaches DRAM before the launch ends.
NCU_DRAM_BYTES_PER_WEIGHT_BYTE = 17643264 / 17432576
NCU_LMHEAD_LOGIT_WRITE_FRACTION = 26198016 / 38895616


def model_dir(shape: str, variant: str = "") -> str:
    name = f"tffn_bench_{shape}" + (f"_{variant}" if variant else "")
    for base in ("/dev/shm", "/tmp"):  # an existing copy wins; else the first place with room
        if os.path.exists(os.path.join(base, name, ".complete")):
            return os.path.join(base, name)
    base = "/dev/shm" if os.path.isdir("/dev/shm") and shutil.disk_usage("/dev/shm").free > (40 << 30) else "/tmp"
    return os.path.join(base, name)


def ensure_model(shape: str, variant: str = "") -> tuple[str, str, dict]:
    """Seeded synthetic model dir + expert .bin of the shape, written once per machine. variant "peaked":
    vocabulary rows with log-normal norms (synth.write_model head_norm_sigma), whose logits have a clear
    winner; used by the parity tests that assert raw top-1 agreement."""
    import synth
    d = model_dir(shape, variant)
    ep = os.path.join(d, "expert.bin")
    marker = os.path.join(d, ".complete")
    if not os.path.exists(marker):
        shutil.rmtree(d, ignore_errors=True)
        fast = shape == "7b"  # 38 GB of files: cut out of one random block, only the sizes matter for throughput
        cfg = synth.write_model(d, shape, seed=1234, head_norm_sigma=1.5 if variant == "peaked" else 0.0, fast=fast)
        synth.write_expert(ep, cfg, seed=4321, fast=fast)
        with open(marker, "w") as f:
            f.write("ok")
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return d, ep, cfg


class ClockSampler:
    """nvidia-smi samples (read-only) of SM clock, power and throttle reasons while the timed regions run."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_uuid: str | None):
        self.rows, self.proc, self.thread = [], None, None
        cmd = ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50"]
        if gpu_uuid:
            cmd += ["-i", gpu_uuid]
        try:
            self.proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1])); pw.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        load = [s for s, p in zip(sm, pw) if p >= 0.5 * max(pw)] or sm
        return {"sm_mhz": float(np.median(load)), "sm_max_mhz": float(max(mx)), "power_w_max": float(max(pw)),
                "samples": len(sm), "reasons": sorted(reasons)}


def kernel_bytes(cfg: dict, with_expert: bool, n_seqs: int, ctx: float, head_dim: int | None = None) -> dict:
    """Algorithmic HBM bytes per decode step, per kernel class: every weight matrix once per step,
    the KV cache of every sequence once per layer. Activations, partial sums and logits are not credited."""
    H, I, L, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = head_dim or H // nh
    nqkv = (nh + 2 * nkv) * hd
    ffn = 3 * I * H * 2 * (2 if with_expert else 1)
    kv = n_seqs * 2 * nkv * hd * 2 * (ctx + 1)  # K and V rows of the context plus the new row
    b = {
        "gemm_tc:qkv": L * nqkv * H * 2, "gemm_tc:o_proj": L * H * nh * hd * 2,
        "gemm_tc:gate_up_swiglu": L * ffn * 2 // 3, "gemm_tc:down": L * ffn // 3, "gemm_tc:lm_head": V * H * 2,
        "attn_decode": L * kv,
        "bs1_qkv": L * nqkv * H * 2, "bs1_oproj": L * H * nh * hd * 2, "bs1_ffn": L * ffn, "bs1_lmhead": V * H * 2,
    }
    return b


def dp_sequence_ids(rank: int, seqs_per_rank: int) -> list[int]:
    """Data-parallel sharding: rank r owns the global sequences [r*n, (r+1)*n); no sequence is shared
    and nothing is exchanged on the data path."""
    return list(range(rank * seqs_per_rank, (rank + 1) * seqs_per_rank))


def dp_prompts(rank: int, seqs_per_rank: int, prompt_len: int):
    import synth
    ids = dp_sequence_ids(rank, seqs_per_rank)
    return synth.prompts(len(ids), prompt_len, 1, first_seq=ids[0])


def reduce_max(dist, x: float, device: str) -> float:
    """max over ranks of a per-rank device time (the job is as slow as its slowest rank)"""
    if dist is None:
        return x
    import torch
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def timed_decode(sess, stream, n, K, reps, barrier, max_over_ranks, want_tokens=False):
    """K device-resident decode steps, repeated `reps` times; each repetition is bracketed by a barrier and a
    synchronize on both sides and timed with CUDA events on the launching stream. Returns (median ms over
    the repetitions after the max over ranks, all ms, tokens of the first repetition, launches per repetition)."""
    import torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times, toks, launches = [], None, 0
    for r in range(reps):
        barrier()
        l0 = sess.launch_count()
        e0.record(stream)
        t = sess.decode_run(n, K, want_tokens=want_tokens and r == 0)
        e1.record(stream)
        barrier()
        if r == 0:
            toks, launches = t, sess.launch_count() - l0
        times.append(max_over_ranks(e0.elapsed_time(e1)))
    return float(np.median(times)), times, toks, launches


def reference_bs1(d: str, ep: str, prompt_len: int, n_tokens: int, reps: int):
    """The reference's own decode loop (oracle/_ref/ref_driver: its unmodified sources) at configs[0]'s shape of
    work: one sequence, prompt_len-token prompt, n_tokens greedy tokens, with the expert."""
    import synth
    drv = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
    if not os.path.exists(drv):
        return None
    toks = synth.prompts(1, prompt_len, 0)[0]
    tf = os.path.join(os.path.dirname(ep), "ref_bs1_tokens.i32")
    toks.tofile(tf)
    out = os.path.join(os.path.dirname(ep), "ref_bs1_out")
    try:
        subprocess.check_call([drv, "--model", d, "--expert", ep, "--expert-scale", "0.1", "--max-seq",
                               str(prompt_len + n_tokens + 8), "--tokens", tf, "--prompt-len", str(prompt_len), "--new",
                               str(n_tokens), "--out", out, "--time", str(reps)], stdout=subprocess.DEVNULL)
        with open(out + ".time.json") as f:
            t = json.load(f)
    except Exception as ex:
        return {"error": str(ex)}
    return {"tok_s_best": n_tokens / (t["decode_ms_best"] / 1e3), "tok_s_mean": n_tokens / (t["decode_ms_mean"] / 1e3),
            "reps": reps, "prompt_len": prompt_len, "new_tokens": n_tokens,
            "what": "the reference's unmodified CUDA sources, its own loop (token H2D, forward, logits D2H, host argmax)"}


def run_ours(a):
    import torch
    import synth
    import tffn

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        if world == 1 and a.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
    tp_size = a.tp if a.tp > 1 else 1
    if tp_size > 1 and tp_size != world:
        raise SystemExit("--tp N needs exactly N ranks (torchrun --nproc-per-node N ... --gpus N --tp N)")
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x: float) -> float:
        return reduce_max(dist, x, "cuda")

    if rank == 0:
        ensure_model(a.shape)
    barrier()
    d, ep, cfg = ensure_model(a.shape)
    K, W, n = a.steps, a.warmup, a.seqs
    reps = a.reps if a.reps > 0 else max(1, min(10, 256 // max(K, 1)))
    max_seq = a.prompt + W + K * reps + 8 + 16  # + the per-kernel profile pass and the timeline steps
    stream = torch.cuda.Stream(device=local)
    group = None
    if tp_size > 1:
        meet = os.path.join("/tmp", f"tffn_tp_meet_{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}")
        group = tffn.TpGroup(tffn.tp_rendezvous(meet, rank, tp_size, 300.0), rank, tp_size, local)
    model = tffn.qwen_load(d, device=local, tp_rank=rank if tp_size > 1 else 0, tp_size=tp_size)
    expert = tffn.checkpoint_load(ep, model, 0.1)
    sess = tffn.Session(model, expert, max_batch=n, max_seq=max_seq, stream=stream.cuda_stream, tp=group)
    sess.set_launch_mode(a.launch_mode)
    if tp_size > 1 and a.tp_nccl:
        sess.set_tp_fused(False)
    # data parallel: distinct sequences on every rank; tensor parallel: the same sequences on every rank
    prompts = dp_prompts(0 if tp_size > 1 else rank, n, a.prompt)
    prompt_list = [prompts[i] for i in range(n)]

    uuid = None
    try:
        uuid = str(torch.cuda.get_device_properties(local).uuid)
        if not uuid.startswith("GPU-"):
            uuid = "GPU-" + uuid
    except Exception:
        pass
    sampler = ClockSampler(uuid) if rank == 0 else None

    # ---- device-resident decode (value)
    t0 = time.perf_counter()
    sess.prefill(prompt_list)
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    sess.decode_run(n, W, want_tokens=False)
    ms, rep_ms, toks_dev, launches = timed_decode(sess, stream, n, K, reps, barrier, max_over_ranks, want_tokens=True)
    groups = 1 if tp_size > 1 else world
    value = groups * n * K / (ms / 1e3)

    # ---- per-kernel device time (separate pass; the event pairs serialise the kernels)
    P = min(8, K)
    sess.profile(True)
    sess.decode_run(n, P, want_tokens=False)
    prof = sess.profile_read()
    sess.profile(False)
    ctx_mid = a.prompt + W + K * reps / 2.0
    cfg_rank = dict(cfg)
    if tp_size > 1:  # this rank's slices
        part = tffn.tp_partition(model.cfg, rank, tp_size)
        cfg_rank.update(num_attention_heads=part["n_q_heads"], num_key_value_heads=part["n_kv_heads"],
                        intermediate_size=part["n_i"], vocab_size=part["n_v"])
    kb = kernel_bytes(cfg_rank, True, n, ctx_mid, head_dim=cfg["hidden_size"] // cfg["num_attention_heads"])
    kernels = []
    for name, (kms, cnt) in sorted(prof.items(), key=lambda kv: -kv[1][0]):
        row = {"kernel": name, "launches_per_step": cnt / P, "ms_per_step": kms / P}
        if name in kb:
            row["algorithmic_gbs"] = kb[name] / 1e9 / (kms / P / 1e3)
        kernels.append(row)
    peak, peak_kind = peaks()
    gemm_ms = sum(v[0] for k, v in prof.items() if k.startswith("gemm_tc:")) / P
    gemm_n = sum(v[1] for k, v in prof.items() if k.startswith("gemm_tc:")) / P
    gemm_bytes = sum(v for k, v in kb.items() if k.startswith("gemm_tc:"))
    serialised = gemm_bytes / 1e9 / (gemm_ms / 1e3) if gemm_ms > 0 else 0.0
    roofline = {"bound": "hbm", "kernel": "k_gemm_tc (all launches of a decode step)", "peak": peak, "peak_kind": peak_kind,
                "unit": "GB/s", "launches_per_step": gemm_n, "algorithmic_bytes_per_launch": gemm_bytes / max(gemm_n, 1),
                # diagnostic only: every launch bracketed by events, which serialises kernels that overlap in the
                # real step and adds the launch gap to each; the sum can exceed the step itself
                "serialised": {"achieved": serialised, "frac": serialised / peak, "avg_launch_us": 1e3 * gemm_ms / max(gemm_n, 1)}}
    # traffic per launch: the captured read ratio applied to this step's weight bytes, plus the logits written
    traffic = gemm_bytes * NCU_DRAM_BYTES_PER_WEIGHT_BYTE + NCU_LMHEAD_LOGIT_WRITE_FRACTION * n * cfg_rank["vocab_size"] * 4
    roofline["traffic"] = a.traffic if a.traffic is not None else traffic / max(gemm_n, 1)
    roofline["traffic_source"] = ("--traffic" if a.traffic is not None else
                                  "ncu capture of two launches (gate|up rows of one layer, LM head), scaled by weight bytes")
    # the step as it runs (graph + dependent launches): per kernel class the time from the previous kernel's
    # last CTA leaving to this kernel's last CTA leaving, from in-kernel globaltimer stamps. The roofline
    # fraction of the dominant kernel is taken from these times.
    in_situ = None
    try:
        names, tl = sess.timeline(n)
        tl = tl.astype(np.int64)
        agg: dict = {}
        prev = int(tl[:, 0].min())
        for nm, r in zip(names, tl):
            e = agg.setdefault(nm, [0, 0.0])
            e[0] += 1
            e[1] += (int(r[5]) - prev) / 1e3
            prev = int(r[5])
        in_situ = {"step_us": (int(tl[:, 5].max()) - int(tl[:, 0].min())) / 1e3,
                   "kernels": [{"kernel": nm, "launches": v[0], "us_per_launch": v[1] / v[0]}
                               for nm, v in sorted(agg.items(), key=lambda kv: -kv[1][1])]}
        # tensor parallel over peer memory: of what the exchange kernel adds to the step, how long the last block
        # waited for its peers after its own dependency wait was over is not in the stamps separately; what is:
        # entry -> hand-shake over (max over blocks) and hand-shake over -> exit
        ex = [(int(r[3]) - int(r[0]), int(r[5]) - int(r[3])) for nm, r in zip(names, tl) if nm == "tp_all_reduce"]
        if ex:
            in_situ["tp_all_reduce_phases_us"] = {"entry_to_handshake_over": sum(x[0] for x in ex) / len(ex) / 1e3,
                                                  "handshake_over_to_exit": sum(x[1] for x in ex) / len(ex) / 1e3}
        gemm_us = sum(v[1] for nm, v in agg.items() if nm.startswith("gemm_tc:"))
        if gemm_us > 0:
            roofline["achieved"] = gemm_bytes / 1e9 / (gemm_us / 1e6)
            roofline["frac"] = roofline["achieved"] / peak
            roofline["avg_launch_us"] = gemm_us / max(gemm_n, 1)
            roofline["timing"] = "in-kernel globaltimer stamps inside the running step"
    except Exception as ex:  # a diagnostic: never fail the bench line for it
        in_situ = {"error": str(ex)}
    if "frac" not in roofline:
        roofline.update(achieved=serialised, frac=serialised / peak, avg_launch_us=1e3 * gemm_ms / max(gemm_n, 1),
                        timing="CUDA events around every launch (serialised)")
    step_bytes = sum(v for k, v in kb.items() if k.startswith("gemm_tc:")) + kb["attn_decode"]
    step_roofline = {"algorithmic_bytes_per_step_per_gpu": step_bytes, "achieved": step_bytes / 1e9 / (ms / K / 1e3),
                     "peak": peak, "unit": "GB/s", "frac": step_bytes / 1e9 / (ms / K / 1e3) / peak}
    tp_info = None
    if tp_size > 1:
        ar = prof.get("tp_all_reduce", (0.0, 0))
        step_prof_ms = sum(v[0] for v in prof.values()) / P
        tp_info = {"tp_size": tp_size,
                   "exchange": "ncclAllReduce (fp32, in place)" if a.tp_nccl else
                   "peer memory: flag hand-shake, then every rank's residual/RMSNorm kernel loads all ranks' fp32 partial sums over NVLink and adds them in rank order",
                   "all_reduce_per_step": ar[1] / P, "all_reduce_us_per_call": 1e3 * ar[0] / max(ar[1], 1),
                   "all_reduce_share_of_serialised_step": (ar[0] / P) / step_prof_ms if step_prof_ms > 0 else None,
                   "all_reduce_bytes": n * cfg["hidden_size"] * 4,
                   "per_rank_roofline_frac": step_roofline["frac"],
                   "per_rank_roofline_frac_without_all_reduce": step_bytes / 1e9 / max(ms / K - ar[0] / P, 1e-6) * 1e3 / peak}
        if in_situ and "kernels" in in_situ:  # what an exchange adds to the running step (peer-memory path only: NCCL kernels carry no stamps)
            for kk in in_situ["kernels"]:
                if kk["kernel"] == "tp_all_reduce":
                    tp_info["all_reduce_us_per_call_in_situ"] = kk["us_per_launch"]
                    tp_info["all_reduce_share_of_step_in_situ"] = kk["us_per_launch"] * kk["launches"] / in_situ["step_us"]

    # ---- end to end through the C ABI with host buffers (e2e)
    e2e = None
    if not a.no_e2e:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sess.qwen_reset()
        nxt, _ = sess.prefill(prompt_list)
        for _ in range(W):
            nxt, _ = sess.decode_step(nxt)
        e2e_times = []
        for _ in range(reps):
            barrier()
            e0.record(stream)
            w0 = time.perf_counter()
            for _ in range(K):
                nxt, _ = sess.decode_step(nxt)  # host int32[n] in, host int32[n] out, every step
            e1.record(stream)
            barrier()
            wall_ms = (time.perf_counter() - w0) * 1e3
            e2e_times.append(max_over_ranks(max(e0.elapsed_time(e1), wall_ms)))
        e2e_ms = float(np.median(e2e_times))
        e2e = {"value": groups * n * K / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 4 * n * world,
               "d2h_bytes_per_step": 4 * n * world, "ms_per_step": e2e_ms / K, "repetitions": reps}

    # ---- data parallel at N > 1: every rank's tokens are checked, and 64 sequences in total (strong scaling)
    dp_check, strong = None, None
    if dist is not None and tp_size == 1:
        mine = np.ascontiguousarray(np.asarray(toks_dev, dtype=np.int32))
        sums = [None] * world
        dist.all_gather_object(sums, int(mine.astype(np.int64).sum()))
        other = 1 % world
        box = [mine.tolist() if rank == other else None]
        dist.broadcast_object_list(box, src=other)
        same = None
        if rank == 0:  # rank 0 decodes rank `other`'s shard itself: the tokens must be the same, bit for bit
            s2 = tffn.Session(model, expert, max_batch=n, max_seq=a.prompt + W + K + 8, stream=stream.cuda_stream)
            s2.set_launch_mode(a.launch_mode)
            p2 = dp_prompts(other, n, a.prompt)
            s2.prefill([p2[i] for i in range(n)])
            s2.decode_run(n, W, want_tokens=False)
            t2 = np.asarray(s2.decode_run(n, K, want_tokens=True), dtype=np.int32)
            same = bool((t2 == np.asarray(box[0], dtype=np.int32).reshape(t2.shape)).all())
            s2.free()
        barrier()
        dp_check = {"checksum_tokens_per_rank": sums, "rank0_reran_rank": other, "identical_tokens": same}
        if n % world == 0 and n // world >= 1:
            ns = n // world
            s3 = tffn.Session(model, expert, max_batch=ns, max_seq=a.prompt + W + K * reps + 8, stream=stream.cuda_stream)
            s3.set_launch_mode(a.launch_mode)
            p3 = synth.prompts(ns, a.prompt, 1, first_seq=rank * ns)  # global sequences [rank*ns, (rank+1)*ns)
            s3.prefill([p3[i] for i in range(ns)])
            s3.decode_run(ns, W, want_tokens=False)
            ms3, _, _, _ = timed_decode(s3, stream, ns, K, reps, barrier, max_over_ranks)
            kb3 = kernel_bytes(cfg, True, ns, ctx_mid)
            b3 = sum(v for k, v in kb3.items() if k.startswith("gemm_tc:")) + kb3["attn_decode"]
            strong = {"value": n * K / (ms3 / 1e3), "unit": "tok/s", "total_sequences": n, "sequences_per_gpu": ns,
                      "ms_per_step": ms3 / K, "per_gpu_roofline_frac": b3 / 1e9 / (ms3 / K / 1e3) / peak,
                      "note": "every GPU still streams all weights per step: the aggregate HBM roofline grows only ~1.3x from 1 to 8 GPUs at 64 sequences"}
            s3.free()

    # ---- batch 1 (configs[0]) on the same weights: 128-token prompt, greedy decode
    bs1 = None
    if not a.no_bs1 and tp_size == 1:
        s1 = tffn.Session(model, expert, max_batch=1, max_seq=128 + W + a.bs1_steps * 4 + 24, stream=stream.cuda_stream)
        s1.set_launch_mode(a.launch_mode)
        p1 = synth.prompts(1, 128, 0)[0]
        s1.prefill([p1])
        s1.decode_run(1, W, want_tokens=False)
        ms1, _, _, l1 = timed_decode(s1, stream, 1, a.bs1_steps, 3, barrier, max_over_ranks)
        s1.profile(True)
        s1.decode_run(1, 8, want_tokens=False)
        prof1 = s1.profile_read()
        s1.profile(False)
        ctx1 = 128 + W + a.bs1_steps * 1.5
        kb1 = kernel_bytes(cfg, True, 1, ctx1)
        tok_bytes = kb1["bs1_qkv"] + kb1["bs1_oproj"] + kb1["bs1_ffn"] + kb1["bs1_lmhead"] + kb1["attn_decode"]
        bs1 = {"value": world * a.bs1_steps / (ms1 / 1e3), "unit": "tok/s", "ms_per_token": ms1 / a.bs1_steps,
               "steps": a.bs1_steps, "repetitions": 3, "launch_mode": a.launch_mode, "gpu_launches": l1,
               "algorithmic_bytes_per_token": tok_bytes,
               "roofline_frac_token": tok_bytes / 1e9 / (ms1 / a.bs1_steps / 1e3) / peak,
               "kernels_serialised": [{"kernel": k, "ms_per_token": v[0] / 8, "launches_per_token": v[1] / 8}
                                      for k, v in sorted(prof1.items(), key=lambda kv: -kv[1][0])]}
        try:  # the token as it runs: what each kernel class adds to it (in-kernel stamps, no event pairs)
            names1, tl1 = s1.timeline(1)
            tl1 = tl1.astype(np.int64)
            agg1: dict = {}
            prev = int(tl1[:, 0].min())
            for nm, r in zip(names1, tl1):
                e = agg1.setdefault(nm, [0, 0.0])
                e[0] += 1
                e[1] += (int(r[5]) - prev) / 1e3
                prev = int(r[5])
            bs1["kernels_in_situ"] = {"token_us": (int(tl1[:, 5].max()) - int(tl1[:, 0].min())) / 1e3,
                                      "kernels": [{"kernel": nm, "launches": v[0], "us_per_launch": v[1] / v[0]}
                                                  for nm, v in sorted(agg1.items(), key=lambda kv: -kv[1][1])]}
            ffn_us = agg1.get("bs1_ffn", [0, 0.0])[1]
            if ffn_us > 0:
                bs1["dominant_kernel"] = {"kernel": "k_bs1_ffn", "us_per_token": ffn_us,
                                          "achieved_gbs": kb1["bs1_ffn"] / 1e9 / (ffn_us / 1e6),
                                          "frac": kb1["bs1_ffn"] / 1e9 / (ffn_us / 1e6) / peak}
        except Exception as ex:
            bs1["kernels_in_situ"] = {"error": str(ex)}
        s1.free()
        if rank == 0 and world == 1 and not a.no_ref_bs1:
            bs1["reference"] = reference_bs1(d, ep, 128, a.bs1_steps, 3)
            if bs1["reference"] and "tok_s_best" in bs1["reference"]:
                bs1["speedup_vs_reference_same_config"] = bs1["value"] / bs1["reference"]["tok_s_best"]

    clocks = sampler.stop() if sampler else None

    # ---- CPU baseline: the oracle (a port: the reference has no CPU path), rank 0, one GPU only
    cpu = None
    if rank == 0 and world == 1 and not a.no_cpu:
        cpu = cpu_baseline(d, ep, a.cpu_prompt if a.cpu_prompt > 0 else a.prompt, a.cpu_tokens)

    if rank == 0:
        weights_mb = model.weight_bytes(True) / 1e6
        line = {
            "metric": metric_name(a), "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong" if tp_size > 1 else "weak",
            "vs_baseline": None, "dtype": "bf16",
            "data": f"synthetic (seeded random-init weights of the {a.shape} shape + dense N(0,0.02) expert; uniform-random prompts)",
            "config": {"workload": workload_name(a), "seqs_per_gpu": n if tp_size == 1 else None,
                       "seqs_total": n * groups, "prompt_len": a.prompt, "decode_steps": K, "repetitions": reps,
                       "rep_ms": rep_ms,
                       "parallelism": f"tp{tp_size} (fp32 all-reduce after o_proj and after the FFN)" if tp_size > 1 else f"dp{world} (no collective)",
                       "l2": f"no flush: each step streams {weights_mb:.0f} MB of weights per GPU + KV, more than the 126 MB L2"},
            "e2e": e2e, "gpu_launches": int(launches) * reps, "roofline": roofline, "step_roofline": step_roofline,
            "kernels": kernels, "kernels_in_situ": in_situ, "clocks": clocks, "cpu_baseline": cpu, "prefill_s": prefill_s,
            "checksum_tokens": int(np.asarray(toks_dev, dtype=np.int64).sum()),
        }
        if bs1:
            line["bs1"] = bs1
        if tp_info:
            line["tp"] = tp_info
        if dp_check:
            line["dp_check"] = dp_check
        if strong:
            line["strong_scaling"] = strong
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def cpu_baseline(d: str, ep: str, prompt_len: int, n_tokens: int) -> dict:
    """Times oracle/ (the scalar C++ restatement, OpenMP over output rows) on the host cores: one
    sequence, greedy decode, like the reference's own loop (which has no batching)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    import synth
    o = oracle.Oracle(d, prompt_len + n_tokens + 2, ep, 0.1)
    p = synth.prompts(1, prompt_len, 0)[0]
    nxt = int(o.forward(p, want_logits=False, last_only=True)["argmax"][0])
    t0 = time.perf_counter()
    for _ in range(n_tokens):
        nxt = int(o.forward([nxt], want_logits=False, last_only=True)["argmax"][0])
    dt = time.perf_counter() - t0
    return {"value": n_tokens / dt, "unit": "tok/s", "cores": o.threads, "kind": "port",
            "sample": f"1 sequence of the workload, {prompt_len}-token prompt (untimed) then {n_tokens} greedy tokens (timed); "
                      "the reference decodes sequences one at a time, so its tok/s does not depend on the batch"}


def run_reference(a):
    """The reference's own implementation of the path. It is CUDA-only (no CPU compute path), so
    the compiled reference (oracle/_ref/ref_driver: its unmodified sources + a token-file driver)
    runs on the GPU when one is present; otherwise the CPU port is timed. It has no batching: one of the
    workload's sequences is decoded, K tokens per repetition, the same number of repetitions as this
    library's arm, median over the repetitions."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import synth
    d, ep, cfg = ensure_model(a.shape)
    drv = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
    K, W = a.steps, a.warmup
    reps = a.reps if a.reps > 0 else max(1, min(10, 256 // max(K, 1)))
    have_gpu = shutil.which("nvidia-smi") is not None and subprocess.call(
        ["nvidia-smi", "-L"], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) == 0
    base = {"metric": metric_name(a), "unit": "tok/s", "n_gpus": a.gpus, "steps": K, "warmup": W, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "reference", "data": "synthetic",
            "config": {"workload": workload_name(a), "seqs_per_gpu": a.seqs, "prompt_len": a.prompt, "decode_steps": K,
                       "repetitions": reps,
                       "same_config": False,
                       "note": "the reference decodes one sequence at a time (no batching): one of the workload's sequences is timed"}}
    if os.path.exists(drv) and have_gpu and cfg["num_hidden_layers"] <= 32:
        toks = synth.prompts(1, a.prompt, 1000)[0]
        tf = os.path.join(model_dir(a.shape), "ref_tokens.i32")
        toks.tofile(tf)
        out = os.path.join(model_dir(a.shape), "ref_out")
        # the repetitions run inside one start of the driver (--time): it reloads the model each time it is started
        subprocess.check_call([drv, "--model", d, "--expert", ep, "--expert-scale", "0.1", "--max-seq",
                               str(a.prompt + K + W + 8), "--tokens", tf, "--prompt-len", str(a.prompt), "--new",
                               str(K), "--out", out, "--time", str(reps + 1)], stdout=subprocess.DEVNULL)
        with open(out + ".time.json") as f:
            t = json.load(f)
        v = K / (t["decode_ms_mean"] / 1e3)
        line = dict(base, value=v, ms_per_step=t["decode_ms_mean"] / K, value_best_repetition=K / (t["decode_ms_best"] / 1e3),
                    cpu_baseline={"value": v, "unit": "tok/s", "cores": 1, "kind": "reference",
                                  "sample": f"the reference's unmodified CUDA sources compiled for sm_100 (it has no CPU "
                                            f"path), its own loop: 1 of the {a.seqs} sequences, {a.prompt}-token prompt, "
                                            f"{K} greedy tokens, mean of {reps + 1} repetitions"},
                    e2e={"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    else:
        c = cpu_baseline(d, ep, min(a.prompt, a.cpu_prompt if a.cpu_prompt > 0 else a.prompt), min(K, a.cpu_tokens))
        line = dict(base, value=c["value"], ms_per_step=1e3 / c["value"], cpu_baseline=c,
                    e2e={"value": c["value"], "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    print(json.dumps(line), flush=True)


def run_kernel_case(a):
    """k_gemm_tc alone, one launch per shape, inputs seeded: [64 tokens] x [gate|up rows of one layer]
    (17 MB of weights, cold: what every layer's launch sees in a step that cycles 1 GB through L2) and
    x [vocabulary rows] (272 MB, larger than L2). Prints one JSON line with the wall time of each call
    (host copies included, so not a kernel time)."""
    import synth
    import tffn
    cfg = synth.SHAPES[a.shape] if hasattr(synth, "SHAPES") else None
    H = cfg["hidden_size"] if isinstance(cfg, dict) else 896
    I = cfg["intermediate_size"] if isinstance(cfg, dict) else 4864
    V = cfg["vocab_size"] if isinstance(cfg, dict) else 151936
    rng = np.random.default_rng(7)
    X = synth.f32_to_bf16(rng.standard_normal((a.seqs, H), dtype=np.float32))
    out = {"kernel_case": "gemm", "tokens": a.seqs, "K": H, "cases": []}
    for name, N in (("gate_up_rows", 2 * I), ("lm_head", V)):
        W = synth.f32_to_bf16((rng.standard_normal((N, H), dtype=np.float32) * 0.02))
        t0 = time.perf_counter()
        y = tffn.op_gemm(X, W)
        dt = time.perf_counter() - t0
        ref = synth.bf16_to_f32(X[:2]) @ synth.bf16_to_f32(W[:256]).T
        err = float(np.abs(y[:2, :256] - ref).max())
        out["cases"].append({"name": name, "N": N, "weight_bytes": int(N) * H * 2, "out_bytes": a.seqs * int(N) * 4,
                             "call_s": dt, "max_abs_err_vs_numpy_sample": err})
    print(json.dumps(out))


def run_expert_forward_case(a):
    """tffn_expert_forward (the trainer's expert_forward on the inference kernels) on a training-shaped
    batch of the bench model: 4096 tokens per layer, all layers; prints dense bf16 TFLOP/s against the
    measured GEMM peak (a tensor-bound case, unlike the decode path)."""
    import torch
    import synth
    import tffn
    d, ep, cfg = ensure_model(a.shape)
    H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
    T = 4096
    model = tffn.qwen_load(d, device=0)
    expert = tffn.checkpoint_load(ep, model, 0.01)
    x = torch.randn((L, T, H), device="cuda", dtype=torch.float32).to(torch.bfloat16)
    out = torch.empty((L, T, H), device="cuda", dtype=torch.float32)
    for _ in range(3):
        expert.expert_forward(x.data_ptr(), out.data_ptr(), T)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 5
    e0.record()
    for _ in range(reps):
        expert.expert_forward(x.data_ptr(), out.data_ptr(), T)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    flops = 6.0 * L * T * H * I
    peak = None
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            peak = float(json.load(f).get("bf16_tflops", 0)) or None
    tf = flops / (ms / 1e3) / 1e12
    print(json.dumps({"kernel_case": "expert_forward", "layers": L, "batch_tokens": T, "hidden": H, "intermediate": I,
                      "ms": ms, "tflops": tf, "peak_tflops": peak, "peak_kind": "measured" if peak else None,
                      "frac": tf / peak if peak else None, "finite": bool(torch.isfinite(out).all().item())}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="0.5b")
    ap.add_argument("--seqs", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--bs1-steps", type=int, default=128)
    ap.add_argument("--launch-mode", type=int, default=2)
    ap.add_argument("--no-bs1", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer loop (profiling runs)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--cpu-prompt", type=int, default=0, help="prompt length of the CPU baseline (0: the workload's)")
    ap.add_argument("--cpu-tokens", type=int, default=64)
    ap.add_argument("--reps", type=int, default=0, help="repetitions of the timed region (0: as many as fit 256 steps, at most 10)")
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel group size (= number of ranks); 1: data parallel")
    ap.add_argument("--tp-nccl", action="store_true", help="with --tp: every all-reduce through NCCL instead of the peer windows")
    ap.add_argument("--no-ref-bs1", action="store_true", help="skip the reference run at the batch-1 configuration")
    ap.add_argument("--kernel-case", default="", choices=["", "gemm", "expert_forward"],
                    help="run only the tensor-core GEMM on the decode step's two largest shapes (gate|up rows, LM head) "
                         "through the op-level entry point and exit: the small program that ncu captures are taken from")
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch of the dominant kernel from an ncu capture, if known")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)
    if a.kernel_case == "expert_forward":
        run_expert_forward_case(a)
        return
    if a.kernel_case:
        run_kernel_case(a)
        return
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
