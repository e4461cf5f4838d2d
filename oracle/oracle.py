"""TEST INFRASTRUCTURE — Python face of the CPU oracle (oracle/tffn_oracle.cpp).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this.
It has its own readers for the model files so that it shares no code with the product.
"""
from __future__ import annotations

import ctypes
import json
import os
import struct
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "liboracle.so")


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "tffn_oracle.cpp")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.check_call(["g++", "-O3", "-march=x86-64-v3", "-fopenmp", "-fno-fast-math", "-shared",
                               "-fPIC", "-o", LIB, src])
    return LIB


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            build()
        L = ctypes.CDLL(LIB)
        L.oracle_create.restype = ctypes.c_void_p
        L.oracle_create.argtypes = [ctypes.c_int] * 7 + [ctypes.c_float] * 2
        L.oracle_free.argtypes = [ctypes.c_void_p]
        L.oracle_threads.argtypes = [ctypes.c_void_p]
        L.oracle_set_threads.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.oracle_set_global.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
        L.oracle_set_layer.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        L.oracle_set_expert.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_float]
        L.oracle_reset.argtypes = [ctypes.c_void_p]
        L.oracle_kv_len.argtypes = [ctypes.c_void_p]
        L.oracle_forward.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                     ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        L.oracle_f32_to_bf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
        L.oracle_get_kv.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
        _lib = L
    return _lib


def read_safetensors_dir(dirpath: str) -> dict[str, np.ndarray]:
    """name -> uint16 view (BF16 bits) memory-mapped from every *.safetensors in the dir
    (format: inference/src/io/safetensors.cpp:41-78; shards by sorted name :104-118)."""
    out = {}
    for fn in sorted(os.listdir(dirpath)):
        if not fn.endswith(".safetensors"):
            continue
        path = os.path.join(dirpath, fn)
        with open(path, "rb") as f:
            (hl,) = struct.unpack("<Q", f.read(8))
            header = json.loads(f.read(hl))
        mm = np.memmap(path, dtype=np.uint8, mode="r", offset=8 + hl)
        for name, info in header.items():
            if name == "__metadata__" or name in out:
                continue
            assert info["dtype"] == "BF16", (name, info["dtype"])
            s, e = info["data_offsets"]
            out[name] = np.frombuffer(mm, dtype=np.uint16, count=(e - s) // 2, offset=s).reshape(info["shape"])
    return out


def read_expert(path: str):
    """(L, H, I, fp32 memmap [L, 3, I*H]) — format: trainer/include/io/checkpoint.h:12-24."""
    with open(path, "rb") as f:
        magic, version, L, H, I = struct.unpack("<5I", f.read(20))
    if magic != 0x45585054:
        raise ValueError("bad expert magic 0x%08x" % magic)
    data = np.memmap(path, dtype=np.float32, mode="r", offset=20, shape=(L, 3, I * H))
    return L, H, I, data


_LAYER_SLOTS = [
    ("self_attn.q_proj.weight", 0), ("self_attn.k_proj.weight", 1), ("self_attn.v_proj.weight", 2),
    ("self_attn.o_proj.weight", 3), ("self_attn.q_proj.bias", 4), ("self_attn.k_proj.bias", 5),
    ("self_attn.v_proj.bias", 6), ("input_layernorm.weight", 7), ("post_attention_layernorm.weight", 8),
    ("mlp.gate_proj.weight", 9), ("mlp.up_proj.weight", 10), ("mlp.down_proj.weight", 11),
]


class Oracle:
    """One sequence at a time, like the reference's QwenModel (inference/include/model/qwen.h:59-99)."""

    def __init__(self, model_dir: str, max_seq: int = 2048, expert_path: str | None = None,
                 expert_scale: float = 0.1, threads: int = 0):
        L = lib()
        with open(os.path.join(model_dir, "config.json")) as f:
            c = json.load(f)
        self.cfg = c
        self.H, self.I = c.get("hidden_size", 896), c.get("intermediate_size", 4864)
        self.L, self.nh = c.get("num_hidden_layers", 24), c.get("num_attention_heads", 14)
        self.nkv, self.V = c.get("num_key_value_heads", 2), c.get("vocab_size", 151936)
        self.hd = self.H // self.nh
        self.max_seq = max_seq
        self._keep = []
        self.h = L.oracle_create(self.H, self.I, self.L, self.nh, self.nkv, self.V, max_seq,
                                 float(c.get("rms_norm_eps", 1e-6)), float(c.get("rope_theta", 1e6)))
        if threads:
            L.oracle_set_threads(self.h, threads)
        t = read_safetensors_dir(model_dir)
        self.tensors = t

        def ptr(a):
            a = np.ascontiguousarray(a)
            self._keep.append(a)
            return a.ctypes.data

        emb = ptr(t["model.embed_tokens.weight"])
        L.oracle_set_global(self.h, 0, emb)
        L.oracle_set_global(self.h, 1, ptr(t["model.norm.weight"]))
        if c.get("tie_word_embeddings", True):
            L.oracle_set_global(self.h, 2, emb)
        else:
            L.oracle_set_global(self.h, 2, ptr(t["lm_head.weight"]))
        for l in range(self.L):
            for suffix, slot in _LAYER_SLOTS:
                name = f"model.layers.{l}.{suffix}"
                if name in t:
                    L.oracle_set_layer(self.h, l, slot, ptr(t[name]))
        if expert_path:
            eL, eH, eI, data = read_expert(expert_path)
            if (eL, eH, eI) != (self.L, self.H, self.I):
                raise ValueError("expert shape mismatch")
            for l in range(self.L):
                for m in range(3):
                    src = np.ascontiguousarray(data[l, m])
                    dst = np.empty(src.size, dtype=np.uint16)
                    L.oracle_f32_to_bf16(src.ctypes.data, dst.ctypes.data, src.size)
                    self._keep.append(dst)
                    L.oracle_set_layer(self.h, l, 12 + m, dst.ctypes.data)
            L.oracle_set_expert(self.h, 1, expert_scale)

    def close(self):
        if self.h:
            lib().oracle_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def threads(self) -> int:
        return lib().oracle_threads(self.h)

    def set_expert(self, enabled: bool, scale: float = 0.1):
        lib().oracle_set_expert(self.h, int(enabled), scale)

    def reset(self):
        lib().oracle_reset(self.h)

    @property
    def kv_len(self) -> int:
        return lib().oracle_kv_len(self.h)

    def forward(self, tokens, want_logits=True, want_hidden=False, last_only=False):
        """Append tokens; returns dict(logits fp32 [rows,V], hidden uint16 [L,T,H], argmax int32 [rows])."""
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        T = tok.size
        rows = 1 if last_only else T
        logits = np.empty((rows, self.V), dtype=np.float32) if want_logits else None
        hidden = np.empty((self.L, T, self.H), dtype=np.uint16) if want_hidden else None
        am = np.empty(rows, dtype=np.int32)
        rc = lib().oracle_forward(self.h, tok.ctypes.data, T,
                                  logits.ctypes.data if want_logits else None,
                                  hidden.ctypes.data if want_hidden else None,
                                  am.ctypes.data, int(last_only))
        if rc != 0:
            raise RuntimeError(f"oracle_forward failed ({rc})")
        return dict(logits=logits, hidden=hidden, argmax=am)

    def get_kv(self, layer: int):
        n = self.kv_len
        k = np.empty((n, self.nkv, self.hd), dtype=np.uint16)
        v = np.empty((n, self.nkv, self.hd), dtype=np.uint16)
        lib().oracle_get_kv(self.h, layer, k.ctypes.data, v.ctypes.data)
        return k, v

    def generate(self, prompt, n_new: int):
        """Greedy: prefill then n_new single-token forwards (inference/src/main.cpp:172-197,
        without the EOS break). Returns the n_new tokens."""
        self.reset()
        nxt = int(self.forward(prompt, want_logits=False, last_only=True)["argmax"][0])
        out = []
        for _ in range(n_new):
            out.append(nxt)
            nxt = int(self.forward([nxt], want_logits=False, last_only=True)["argmax"][0])
        return np.array(out, dtype=np.int32)


if __name__ == "__main__":
    print(build(force=True))


def expert_forward_ref(x_norm_bf16, gate_bf16, up_bf16, down_bf16, scale):
    """CPU restatement of the trainer's expert_forward for ONE layer (trainer/src/model/ffn_expert.cu:151-175;
    test infrastructure, never on the product path). All matrices as bf16 bit patterns (uint16):
    x_norm [T,H], gate/up [I,H], down [H,I]. gemm_bf16_out rounds the fp32 accumulators of gate and up to
    bf16 (:162-165), silu_mul_bf16 forms bf16(silu(g) * u) in fp32 (:166), gemm_bf16 keeps the down
    projection in fp32 (:167-169) and scale_fp32 multiplies it by the output scale (:171). Returns fp32 [T,H]."""
    import numpy as np

    def f32(u):
        return (np.asarray(u).astype(np.uint32) << 16).view(np.float32)

    def bf16r(a):  # round to nearest even to bf16, back to fp32
        b = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
        r = ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint32) << 16
        return r.view(np.float32)

    x = f32(x_norm_bf16)
    g = bf16r(x @ f32(gate_bf16).T)
    u = bf16r(x @ f32(up_bf16).T)
    act = bf16r((g / (1.0 + np.exp(-g.astype(np.float64))).astype(np.float32)) * u)
    return (act @ f32(down_bf16).T).astype(np.float32) * np.float32(scale)
