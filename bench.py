#!/usr/bin/env python
"""Decode throughput of the Qwen2.5 + expert-FFN inference path on B200.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...  # the reference's own code

Workload (BASELINE.json configs[1]): Qwen2.5-0.5B shape + expert, bf16, 64 independent
sequences per GPU, 512-token uniform-random prompts, greedy decode. A "step" is one decode step
of the whole batch (64 new tokens per GPU). With N > 1 the sequences are sharded data-parallel,
64 per rank, no collective on the data path (weak scaling). Weights are seeded synthetic
stand-ins with the real shapes, written to disk in the reference's file formats and loaded
through the library's loader. One JSON line is printed by rank 0.

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
METRIC = "decode tok/s, Qwen2.5-0.5B+expert bf16 bs64 (bs1 in extras); % of HBM roofline"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


# DRAM traffic of k_gemm_tc from the ncu capture summarised in profiles/ncu_gemm_tc_decode_shapes.md
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
        cfg = synth.write_model(d, shape, seed=1234, head_norm_sigma=1.5 if variant == "peaked" else 0.0)
        synth.write_expert(ep, cfg, seed=4321)
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


def kernel_bytes(cfg: dict, with_expert: bool, n_seqs: int, ctx: float) -> dict:
    """Algorithmic HBM bytes per decode step, per kernel class: every weight matrix once per step,
    the KV cache of every sequence once per layer. Activations, partial sums and logits are not credited."""
    H, I, L, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"], cfg["vocab_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = H // nh
    nqkv = (nh + 2 * nkv) * hd
    ffn = 3 * I * H * 2 * (2 if with_expert else 1)
    kv = n_seqs * 2 * nkv * hd * 2 * (ctx + 1)  # K and V rows of the context plus the new row
    b = {
        "gemm_tc:qkv": L * nqkv * H * 2, "gemm_tc:o_proj": L * H * H * 2,
        "gemm_tc:gate_up_swiglu": L * ffn * 2 // 3, "gemm_tc:down": L * ffn // 3, "gemm_tc:lm_head": V * H * 2,
        "attn_decode": L * kv,
        "bs1_qkv": L * nqkv * H * 2, "bs1_oproj": L * H * H * 2, "bs1_ffn": L * ffn, "bs1_lmhead": V * H * 2,
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


def run_ours(a):
    import torch
    import synth
    import tffn

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus:
        if world == 1 and a.gpus > 1:
            raise SystemExit("for --gpus N > 1 launch with: python -m torch.distributed.run --nproc-per-node N bench.py --gpus N ...")
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
    max_seq = a.prompt + W + K + 8 + 16  # + the per-kernel profile pass and the timeline steps
    stream = torch.cuda.Stream(device=local)
    model = tffn.qwen_load(d, device=local)
    expert = tffn.checkpoint_load(ep, model, 0.1)
    sess = tffn.Session(model, expert, max_batch=n, max_seq=max_seq, stream=stream.cuda_stream)
    sess.set_launch_mode(a.launch_mode)
    prompts = dp_prompts(rank, n, a.prompt)  # distinct sequences on every rank
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
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = sess.launch_count()
    e0.record(stream)
    toks_dev = sess.decode_run(n, K, want_tokens=True)
    e1.record(stream)
    barrier()
    launches = sess.launch_count() - launches0
    ms = max_over_ranks(e0.elapsed_time(e1))
    value = world * n * K / (ms / 1e3)

    # ---- per-kernel device time (separate pass; the event pairs serialise the kernels)
    P = min(8, K)
    sess.profile(True)
    sess.decode_run(n, P, want_tokens=False)
    prof = sess.profile_read()
    sess.profile(False)
    ctx_mid = a.prompt + W + K / 2.0
    kb = kernel_bytes(cfg, True, n, ctx_mid)
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
    achieved = gemm_bytes / 1e9 / (gemm_ms / 1e3) if gemm_ms > 0 else 0.0
    roofline = {"bound": "hbm", "kernel": "k_gemm_tc (all launches of a decode step)", "achieved": achieved,
                "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                "launches_per_step": gemm_n, "avg_launch_us": 1e3 * gemm_ms / max(gemm_n, 1),
                "algorithmic_bytes_per_launch": gemm_bytes / max(gemm_n, 1)}
    # traffic per launch: the captured ratio applied to this step's weight bytes, plus the logits written
    traffic = gemm_bytes * NCU_DRAM_BYTES_PER_WEIGHT_BYTE + NCU_LMHEAD_LOGIT_WRITE_FRACTION * n * cfg["vocab_size"] * 4
    roofline["traffic"] = a.traffic if a.traffic is not None else traffic / max(gemm_n, 1)
    roofline["traffic_source"] = ("--traffic" if a.traffic is not None else
                                  "ncu capture of two launches (profiles/ncu_gemm_tc_decode_shapes.md), scaled by weight bytes")
    # the same step as it runs (graph + dependent launches): per kernel class the time from the previous
    # kernel's last CTA leaving to this kernel's last CTA leaving, from in-kernel globaltimer stamps
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
        # the same roofline figure from these in-situ times (no event pairs between the kernels)
        gemm_us = sum(v[1] for nm, v in agg.items() if nm.startswith("gemm_tc:"))
        if gemm_us > 0:
            roofline["achieved_in_situ"] = gemm_bytes / 1e9 / (gemm_us / 1e6)
            roofline["frac_in_situ"] = roofline["achieved_in_situ"] / peak
    except Exception as ex:  # a diagnostic: never fail the bench line for it
        in_situ = {"error": str(ex)}
    step_bytes = sum(v for k, v in kb.items() if k.startswith("gemm_tc:")) + kb["attn_decode"]
    step_roofline = {"algorithmic_bytes_per_step": step_bytes, "achieved": step_bytes / 1e9 / (ms / K / 1e3),
                     "peak": peak, "unit": "GB/s", "frac": step_bytes / 1e9 / (ms / K / 1e3) / peak}

    # ---- end to end through the C ABI with host buffers (e2e)
    e2e = None
    if not a.no_e2e:
        sess.qwen_reset()
        nxt, _ = sess.prefill(prompt_list)
        for _ in range(W):
            nxt, _ = sess.decode_step(nxt)
        barrier()
        e0.record(stream)
        w0 = time.perf_counter()
        for _ in range(K):
            nxt, _ = sess.decode_step(nxt)  # host int32[n] in, host int32[n] out, every step
        e1.record(stream)
        barrier()
        wall_ms = (time.perf_counter() - w0) * 1e3
        e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), wall_ms))
        e2e = {"value": world * n * K / (e2e_ms / 1e3), "unit": "tok/s", "h2d_bytes_per_step": 4 * n * world,
               "d2h_bytes_per_step": 4 * n * world, "ms_per_step": e2e_ms / K}

    # ---- batch 1 (configs[0]) on the same weights: 128-token prompt, greedy decode
    bs1 = None
    if not a.no_bs1:
        s1 = tffn.Session(model, expert, max_batch=1, max_seq=128 + W + a.bs1_steps + 8, stream=stream.cuda_stream)
        s1.set_launch_mode(a.launch_mode)
        p1 = synth.prompts(1, 128, 0)[0]
        s1.prefill([p1])
        s1.decode_run(1, W, want_tokens=False)
        barrier()
        l0 = s1.launch_count()
        e0.record(stream)
        s1.decode_run(1, a.bs1_steps, want_tokens=False)
        e1.record(stream)
        barrier()
        l1 = s1.launch_count() - l0
        ms1 = max_over_ranks(e0.elapsed_time(e1))
        s1.profile(True)
        s1.decode_run(1, 8, want_tokens=False)
        prof1 = s1.profile_read()
        s1.profile(False)
        ctx1 = 128 + W + a.bs1_steps / 2.0
        kb1 = kernel_bytes(cfg, True, 1, ctx1)
        tok_bytes = kb1["bs1_qkv"] + kb1["bs1_oproj"] + kb1["bs1_ffn"] + kb1["bs1_lmhead"] + kb1["attn_decode"]
        ffn_ms = prof1.get("bs1_ffn", (0, 1))[0] / 8
        bs1 = {"value": world * a.bs1_steps / (ms1 / 1e3), "unit": "tok/s", "ms_per_token": ms1 / a.bs1_steps,
               "steps": a.bs1_steps, "launch_mode": a.launch_mode, "gpu_launches": l1,
               "algorithmic_bytes_per_token": tok_bytes,
               "roofline_frac_token": tok_bytes / 1e9 / (ms1 / a.bs1_steps / 1e3) / peak,
               "dominant_kernel": {"kernel": "k_bs1_ffn", "ms_per_token": ffn_ms,
                                   "achieved_gbs": kb1["bs1_ffn"] / 1e9 / (ffn_ms / 1e3) if ffn_ms else None,
                                   "frac": (kb1["bs1_ffn"] / 1e9 / (ffn_ms / 1e3) / peak) if ffn_ms else None},
               "kernels": [{"kernel": k, "ms_per_token": v[0] / 8, "launches_per_token": v[1] / 8}
                           for k, v in sorted(prof1.items(), key=lambda kv: -kv[1][0])]}
        s1.free()

    clocks = sampler.stop() if sampler else None

    # ---- CPU baseline: the oracle (a port: the reference has no CPU path), rank 0, one GPU only
    cpu = None
    if rank == 0 and world == 1 and not a.no_cpu:
        cpu = cpu_baseline(d, ep, a.cpu_prompt, a.cpu_tokens)

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (seeded random-init weights of the Qwen2.5-0.5B shape + dense N(0,0.02) expert; "
                    "uniform-random prompts)",
            "config": {"workload": "configs[1]: Qwen2.5-0.5B+expert, batched greedy decode", "seqs_per_gpu": n,
                       "prompt_len": a.prompt, "decode_steps": K, "parallelism": f"dp{world} (no collective)",
                       "l2": "no flush: each step streams 1.6 GB of weights + KV, far more than the 126 MB L2"},
            "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline, "step_roofline": step_roofline,
            "kernels": kernels, "kernels_in_situ": in_situ, "clocks": clocks, "cpu_baseline": cpu, "prefill_s": prefill_s,
            "checksum_tokens": int(np.asarray(toks_dev, dtype=np.int64).sum()),
        }
        if bs1:
            line["bs1"] = bs1
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
            "sample": f"1 sequence of the workload, {prompt_len}-token prompt then {n_tokens} greedy tokens; the reference "
                      "decodes sequences one at a time, so its tok/s does not depend on the batch"}


def run_reference(a):
    """The reference's own implementation of the path. It is CUDA-only (no CPU compute path), so
    the compiled reference (oracle/_ref/ref_driver: its unmodified sources + a token-file driver)
    runs on the GPU when one is present; otherwise the CPU port is timed."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import synth
    d, ep, cfg = ensure_model(a.shape)
    drv = os.path.join(ROOT, "oracle", "_ref", "ref_driver")
    K, W = a.steps, a.warmup
    have_gpu = shutil.which("nvidia-smi") is not None and subprocess.call(
        ["nvidia-smi", "-L"], stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) == 0
    base = {"metric": METRIC, "unit": "tok/s", "n_gpus": a.gpus, "steps": K, "warmup": W, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "reference", "data": "synthetic",
            "config": {"workload": "configs[1]: Qwen2.5-0.5B+expert, batched greedy decode", "seqs_per_gpu": a.seqs,
                       "prompt_len": a.prompt, "decode_steps": K}}
    if os.path.exists(drv) and have_gpu:
        toks = synth.prompts(1, a.prompt, 1000)[0]
        tf = os.path.join(model_dir(a.shape), "ref_tokens.i32")
        toks.tofile(tf)
        out = os.path.join(model_dir(a.shape), "ref_out")
        reps = 3
        subprocess.check_call([drv, "--model", d, "--expert", ep, "--expert-scale", "0.1", "--max-seq",
                               str(a.prompt + K + W + 8), "--tokens", tf, "--prompt-len", str(a.prompt), "--new",
                               str(K), "--out", out, "--time", str(reps + 1)], stdout=subprocess.DEVNULL)
        with open(out + ".time.json") as f:
            t = json.load(f)
        v = K / (t["decode_ms_best"] / 1e3)
        line = dict(base, value=v, ms_per_step=t["decode_ms_best"] / K,
                    cpu_baseline={"value": v, "unit": "tok/s", "cores": 1, "kind": "reference",
                                  "sample": f"the reference's unmodified CUDA sources compiled for sm_100 (it has no CPU "
                                            f"path), its own loop: 1 of the {a.seqs} sequences, {a.prompt}-token prompt, "
                                            f"{K} greedy tokens, best of {reps + 1} repetitions; it has no batching, so "
                                            "the remaining sequences would run one after another at the same rate"},
                    e2e={"value": v, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
    else:
        c = cpu_baseline(d, ep, min(a.prompt, a.cpu_prompt), min(K, a.cpu_tokens))
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
    ap.add_argument("--cpu-prompt", type=int, default=64)
    ap.add_argument("--cpu-tokens", type=int, default=128)
    ap.add_argument("--kernel-case", default="", choices=["", "gemm", "expert_forward"],
                    help="run only the tensor-core GEMM on the decode step's two largest shapes (gate|up rows, LM head) "
                         "through the op-level entry point and exit: the small program that ncu captures are taken from")
    ap.add_argument("--traffic", type=float, default=None,
                    help="DRAM bytes per launch of the dominant kernel from an ncu capture (profiles/), if known")
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
