"""Seeded synthetic model directories in the on-disk formats the inference path reads.

Writes what `tensor-ffn-inference --model DIR [--expert FILE]` expects:

* ``config.json`` with the keys the reference's config reader uses
  (inference/src/model/qwen.cu:21-63),
* ``model.safetensors`` (optionally several shards) with the HF tensor names the
  reference loads (inference/src/model/qwen.cu:90-118), all BF16,
* a small synthetic ``tokenizer.json`` / ``generation_config.json``
  (inference/src/io/tokenizer.cpp:16-84) so the command line can run,
* an expert ``.bin`` in the trainer's checkpoint format
  (trainer/include/io/checkpoint.h:12-24): 20-byte header then per layer
  gate, up, down as little-endian fp32.

No real Qwen2.5 weights exist offline; these random-init stand-ins have the real shapes.
Linear / embedding weights and q/k/v biases ~ N(0, 0.02), RMSNorm weights 1.0 (or
1 + N(0, 0.1) with ``norm_jitter``), expert matrices ~ N(0, 0.02).
"""
from __future__ import annotations

import json
import os
import struct
from concurrent.futures import ThreadPoolExecutor

import numpy as np

EXPERT_MAGIC = 0x45585054

SHAPES = {
    # name: hidden, layers, q heads, kv heads, intermediate, vocab, tied
    "tiny": dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                 intermediate_size=512, vocab_size=1024, tie_word_embeddings=True),
    "tiny128": dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                    intermediate_size=384, vocab_size=640, tie_word_embeddings=False),
    "0.5b": dict(hidden_size=896, num_hidden_layers=24, num_attention_heads=14, num_key_value_heads=2,
                 intermediate_size=4864, vocab_size=151936, tie_word_embeddings=True),
    "1.5b": dict(hidden_size=1536, num_hidden_layers=28, num_attention_heads=12, num_key_value_heads=2,
                 intermediate_size=8960, vocab_size=151936, tie_word_embeddings=True),
    "3b": dict(hidden_size=2048, num_hidden_layers=36, num_attention_heads=16, num_key_value_heads=2,
               intermediate_size=11008, vocab_size=151936, tie_word_embeddings=True),
    "7b": dict(hidden_size=3584, num_hidden_layers=28, num_attention_heads=28, num_key_value_heads=4,
               intermediate_size=18944, vocab_size=152064, tie_word_embeddings=False),
}


def f32_to_bf16(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def bf16_to_f32(u: np.ndarray) -> np.ndarray:
    return (u.astype(np.uint32) << 16).view(np.float32)


def _normal_bf16(seed, n: int, std: float) -> np.ndarray:
    rng = np.random.default_rng(seed)
    out = np.empty(n, dtype=np.uint16)
    step = 1 << 24
    for i in range(0, n, step):
        m = min(step, n - i)
        out[i:i + m] = f32_to_bf16(rng.standard_normal(m, dtype=np.float32) * np.float32(std))
    return out


def make_config(shape: str | dict, **over) -> dict:
    cfg = dict(SHAPES[shape]) if isinstance(shape, str) else dict(shape)
    cfg.setdefault("max_position_embeddings", 32768)
    cfg.setdefault("rms_norm_eps", 1e-6)
    cfg.setdefault("rope_theta", 1000000.0)
    cfg.setdefault("eos_token_id", 151645)
    cfg.setdefault("bos_token_id", 151643)
    cfg.setdefault("model_type", "qwen2")
    cfg.setdefault("torch_dtype", "bfloat16")
    cfg.update(over)
    return cfg


def tensor_specs(cfg: dict, qkv_bias: bool = True):
    """(name, shape, kind) for every tensor, in file order. kind: 'w' normal, 'n' norm weight."""
    H, I = cfg["hidden_size"], cfg["intermediate_size"]
    nh, nkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = H // nh
    V = cfg["vocab_size"]
    specs = [("model.embed_tokens.weight", (V, H), "w")]
    for l in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{l}."
        specs += [
            (p + "self_attn.q_proj.weight", (nh * hd, H), "w"),
            (p + "self_attn.k_proj.weight", (nkv * hd, H), "w"),
            (p + "self_attn.v_proj.weight", (nkv * hd, H), "w"),
            (p + "self_attn.o_proj.weight", (H, nh * hd), "w"),
        ]
        if qkv_bias:
            specs += [
                (p + "self_attn.q_proj.bias", (nh * hd,), "w"),
                (p + "self_attn.k_proj.bias", (nkv * hd,), "w"),
                (p + "self_attn.v_proj.bias", (nkv * hd,), "w"),
            ]
        specs += [
            (p + "input_layernorm.weight", (H,), "n"),
            (p + "post_attention_layernorm.weight", (H,), "n"),
            (p + "mlp.gate_proj.weight", (I, H), "w"),
            (p + "mlp.up_proj.weight", (I, H), "w"),
            (p + "mlp.down_proj.weight", (H, I), "w"),
        ]
    specs.append(("model.norm.weight", (H,), "n"))
    if not cfg.get("tie_word_embeddings", True):
        specs.append(("lm_head.weight", (V, H), "w"))
    return specs


def write_safetensors(path: str, tensors: list[tuple[str, tuple, np.ndarray]]):
    """tensors: (name, shape, uint16 bf16 bits). u64 LE header length | JSON | data."""
    header = {"__metadata__": {"format": "pt"}}
    off = 0
    for name, shape, arr in tensors:
        nbytes = int(arr.size) * 2
        header[name] = {"dtype": "BF16", "shape": list(shape), "data_offsets": [off, off + nbytes]}
        off += nbytes
    hj = json.dumps(header, separators=(",", ":")).encode()
    hj += b" " * ((8 - len(hj) % 8) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for _, _, arr in tensors:
            arr.tofile(f)


def write_tokenizer(dirpath: str, cfg: dict):
    """A tiny vocabulary the reference's naive encoder can use: printable ASCII, the byte-level
    space marker, a few merges, and the ChatML specials at their Qwen ids when they fit."""
    V = cfg["vocab_size"]
    vocab = {}
    for c in range(33, 127):
        vocab[chr(c)] = len(vocab)
    vocab["Ġ"] = len(vocab)  # byte-level BPE's visible space
    merges = []
    for a, b in [("t", "h"), ("i", "n"), ("e", "r"), ("a", "n"), ("th", "e"), ("o", "n"), ("r", "e")]:
        if a in vocab and b in vocab and a + b not in vocab and len(vocab) < V - 8:
            vocab[a + b] = len(vocab)
            merges.append(f"{a} {b}")
    added = []
    specials = [("<|endoftext|>", 151643), ("<|im_start|>", 151644), ("<|im_end|>", 151645)]
    for k, (name, qid) in enumerate(specials):
        tid = qid if qid < V else V - 3 + k
        added.append({"id": tid, "content": name, "special": True})
    tok = {"version": "1.0", "added_tokens": added,
           "model": {"type": "BPE", "vocab": vocab, "merges": merges}}
    with open(os.path.join(dirpath, "tokenizer.json"), "w") as f:
        json.dump(tok, f)
    ids = {a["content"]: a["id"] for a in added}
    with open(os.path.join(dirpath, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": [ids["<|im_end|>"], ids["<|endoftext|>"]],
                   "bos_token_id": ids["<|endoftext|>"]}, f)
    return ids


_TILE = {}


def _tiled_bf16(seed, n: int, std: float) -> np.ndarray:
    """n bf16 values ~ N(0, std) cut out of one seeded 32 Mi-value block at a seed-dependent offset (wrapping
    around): as fast as a copy. For throughput runs on the largest shapes, where only sizes matter."""
    if std not in _TILE:
        _TILE[std] = _normal_bf16([99, int(std * 1e6)], 1 << 25, std)
    blk = _TILE[std]
    off = int(np.random.default_rng(seed).integers(0, blk.size))
    out = np.empty(n, dtype=np.uint16)
    pos = 0
    while pos < n:
        m = min(n - pos, blk.size - off)
        out[pos:pos + m] = blk[off:off + m]
        pos += m
        off = 0
    return out


def write_model(dirpath: str, shape: str | dict = "tiny", seed: int = 1234, qkv_bias: bool = True,
                norm_jitter: float = 0.0, shard_bytes: int = 4 << 30, threads: int = 0, head_norm_sigma: float = 0.0,
                fast: bool = False, **cfg_over) -> dict:
    """head_norm_sigma > 0 gives the vocabulary rows (embedding, and LM head when untied) log-normal
    norms: row v is scaled by exp(head_norm_sigma * z_v). With iid N(0, 0.02) rows the 150 k logits of a
    random-init model are nearly tied somewhere, so that top-1 agreement between two correct
    implementations is decided by rounding noise; with heavy-tailed row norms a few rows compete for the
    maximum and the winner (which still depends on the direction of the final hidden state, i.e. on every
    layer) leads by far more than the bf16 noise."""
    os.makedirs(dirpath, exist_ok=True)
    cfg = make_config(shape, **cfg_over)
    V = cfg["vocab_size"]
    if cfg["eos_token_id"] >= V:
        cfg["eos_token_id"], cfg["bos_token_id"] = V - 1, V - 3
    with open(os.path.join(dirpath, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    write_tokenizer(dirpath, cfg)
    specs = tensor_specs(cfg, qkv_bias)

    def gen(i):
        name, shp, kind = specs[i]
        n = int(np.prod(shp))
        if kind == "n":
            if norm_jitter > 0:
                rng = np.random.default_rng([seed, i])
                return f32_to_bf16(1.0 + norm_jitter * rng.standard_normal(n, dtype=np.float32))
            return f32_to_bf16(np.ones(n, dtype=np.float32))
        if head_norm_sigma > 0 and name in ("model.embed_tokens.weight", "lm_head.weight"):
            rng = np.random.default_rng([seed, i])
            w = rng.standard_normal((shp[0], shp[1]), dtype=np.float32) * np.float32(0.02)
            z = np.random.default_rng([seed, i, 77]).standard_normal(shp[0], dtype=np.float32)
            w *= np.exp(np.float32(head_norm_sigma) * z)[:, None]
            return f32_to_bf16(w.reshape(-1))
        if fast:
            return _tiled_bf16([seed, i], n, 0.02)
        return _normal_bf16([seed, i], n, 0.02)

    threads = threads or min(16, os.cpu_count() or 1)
    # shard by size; generate each shard's tensors in parallel, write, release
    shards, cur, cur_b = [], [], 0
    for i, (name, shp, kind) in enumerate(specs):
        nb = int(np.prod(shp)) * 2
        if cur and cur_b + nb > shard_bytes:
            shards.append(cur)
            cur, cur_b = [], 0
        cur.append(i)
        cur_b += nb
    shards.append(cur)
    with ThreadPoolExecutor(threads) as ex:
        for si, idxs in enumerate(shards):
            arrs = list(ex.map(gen, idxs))
            fn = "model.safetensors" if len(shards) == 1 else f"model-{si + 1:05d}-of-{len(shards):05d}.safetensors"
            write_safetensors(os.path.join(dirpath, fn),
                              [(specs[i][0], specs[i][1], a) for i, a in zip(idxs, arrs)])
            del arrs
    return cfg


def write_expert(path: str, cfg: dict, seed: int = 4321, std: float = 0.02, threads: int = 0,
                 num_layers: int | None = None, hidden: int | None = None, inter: int | None = None,
                 magic: int = EXPERT_MAGIC, truncate_bytes: int = 0, fast: bool = False):
    """Expert checkpoint: u32 magic, version, layers, hidden, intermediate; per layer gate, up, down fp32."""
    L = cfg["num_hidden_layers"] if num_layers is None else num_layers
    H = cfg["hidden_size"] if hidden is None else hidden
    I = cfg["intermediate_size"] if inter is None else inter
    threads = threads or min(16, os.cpu_count() or 1)

    def gen(args):
        l, m = args
        if fast:  # see _tiled_bf16: a seeded block, cut at a per-matrix offset
            return bf16_to_f32(_tiled_bf16([seed, l, m], I * H, std))
        rng = np.random.default_rng([seed, l, m])
        return (rng.standard_normal(I * H, dtype=np.float32) * np.float32(std))

    with open(path, "wb") as f, ThreadPoolExecutor(threads) as ex:
        f.write(struct.pack("<5I", magic, 1, L, H, I))
        group = max(1, threads // 3)
        for l0 in range(0, L, group):
            jobs = [(l, m) for l in range(l0, min(L, l0 + group)) for m in range(3)]
            for arr in ex.map(gen, jobs):
                arr.tofile(f)
    if truncate_bytes:
        with open(path, "r+b") as f:
            f.truncate(max(0, os.path.getsize(path) - truncate_bytes))


def prompts(n_seqs: int, length: int, config_idx: int = 0, vocab_limit: int = 151643, first_seq: int = 0) -> np.ndarray:
    """int32 [n_seqs, length] uniform ids in [0, vocab_limit), one seed per (global) sequence index."""
    out = np.empty((n_seqs, length), dtype=np.int32)
    for s in range(n_seqs):
        rng = np.random.default_rng([2025, config_idx, first_seq + s])
        out[s] = rng.integers(0, vocab_limit, size=length, dtype=np.int32)
    return out


if __name__ == "__main__":
    import argparse
    ap = argparse.ArgumentParser(description="write a seeded synthetic model dir (+ expert .bin)")
    ap.add_argument("--shape", default="tiny", choices=sorted(SHAPES))
    ap.add_argument("--out", required=True)
    ap.add_argument("--expert", default="", help="also write this expert .bin")
    ap.add_argument("--seed", type=int, default=1234)
    a = ap.parse_args()
    c = write_model(a.out, a.shape, seed=a.seed)
    if a.expert:
        write_expert(a.expert, c)
    print(json.dumps(c))
