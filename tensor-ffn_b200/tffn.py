"""ctypes face of libtffn.so (include/tffn.h), shaped like the reference's C++ interface.

The reference's users call free functions over plain structs
(inference/include/model/qwen.h:101-116, expert.h:31-39, io/checkpoint.h:11):

    qwen_load(mdl, dir, max_seq); expert_alloc(...); checkpoint_load(path, expert)
    qwen_forward(mdl, cublas, d_tokens, T, expert_or_null, d_logits); qwen_reset(mdl)

The same names exist here with the same meaning; every error the reference turns into
`exit(1)` is raised as TffnError with the message the library recorded. Nothing in this
module computes on the CPU: if the CUDA library is missing, import fails loudly.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libtffn.so")
kExpertOutputScale = 0.1  # inference/include/model/expert.h:29


class TffnError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"[{code}] {msg}")
        self.code = code
        self.msg = msg


class Config(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("hidden_size", "intermediate_size", "num_layers", "num_heads",
                                              "num_kv_heads", "head_dim", "vocab_size", "max_position_embeddings")] + \
               [("rms_norm_eps", ctypes.c_float), ("rope_theta", ctypes.c_float)] + \
               [(n, ctypes.c_int32) for n in ("eos_token_id", "bos_token_id", "tie_embeddings")]

    def as_dict(self):
        return {n: getattr(self, n) for n, _ in self._fields_}


if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: build it with `python tensor-ffn_b200/build.py` "
                      "(there is no CPU fallback)")
_L = ctypes.CDLL(LIB_PATH)
_vp, _i, _f, _cp = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_char_p
_pp = ctypes.POINTER(ctypes.c_void_p)
_SIGS = {
    "tffn_last_error": (_cp, []),
    "tffn_version": (_i, []),
    "tffn_device_count": (_i, []),
    "tffn_config_read": (_i, [_cp, ctypes.POINTER(Config)]),
    "tffn_expert_probe": (_i, [_cp] + [ctypes.POINTER(ctypes.c_uint32)] * 4),
    "tffn_expert_write": (_i, [_cp, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.POINTER(_vp)]),
    "tffn_safetensors_probe": (_i, [_cp, _cp, ctypes.POINTER(ctypes.c_int32), ctypes.POINTER(ctypes.c_int32), _vp,
                                    ctypes.POINTER(ctypes.c_uint64)]),
    "tffn_tokenizer_load": (_i, [_cp, _pp]),
    "tffn_tokenizer_free": (None, [_vp]),
    "tffn_tokenizer_encode": (_i, [_vp, _cp, _vp, _i]),
    "tffn_tokenizer_decode": (_i, [_vp, _vp, _i, _vp, _i]),
    "tffn_tokenizer_encode_bpe": (_i, [_vp, _cp, _vp, _i]),
    "tffn_tokenizer_decode_bpe": (_i, [_vp, _vp, _i, _vp, _i]),
    "tffn_tokenizer_token_id": (_i, [_vp, _cp, ctypes.POINTER(ctypes.c_uint32)]),
    "tffn_tokenizer_special": (_i, [_vp] + [ctypes.POINTER(ctypes.c_uint32)] * 3),
    "tffn_model_load": (_i, [_cp, _i, _i, _i, _pp]),
    "tffn_model_free": (None, [_vp]),
    "tffn_model_config": (_i, [_vp, ctypes.POINTER(Config)]),
    "tffn_model_weight_bytes": (ctypes.c_uint64, [_vp, _i]),
    "tffn_expert_load": (_i, [_vp, _cp, _f, _pp]),
    "tffn_expert_set_scale": (_i, [_vp, _f]),
    "tffn_expert_get_scale": (_f, [_vp]),
    "tffn_expert_free": (None, [_vp]),
    "tffn_session_create": (_i, [_vp, _vp, _i, _i, _vp, _pp]),
    "tffn_session_free": (None, [_vp]),
    "tffn_session_create_tp": (_i, [_vp, _vp, _i, _i, _vp, _vp, _pp]),
    "tffn_tp_unique_id": (_i, [_vp]),
    "tffn_tp_create": (_i, [_vp, _i, _i, _i, _pp]),
    "tffn_tp_free": (None, [_vp]),
    "tffn_tp_partition": (_i, [ctypes.POINTER(Config), _i, _i, _vp]),
    "tffn_session_reset": (_i, [_vp, _i]),
    "tffn_session_seq_len": (_i, [_vp, _i]),
    "tffn_session_set_launch_mode": (_i, [_vp, _i]),
    "tffn_expert_forward": (_i, [_vp, _vp, _vp, _i, _vp]),
    "tffn_session_set_ablation": (_i, [_vp, ctypes.c_uint]),
    "tffn_session_set_tp_fused": (_i, [_vp, _i]),
    "tffn_session_set_sampling": (_i, [_vp, _f, ctypes.c_uint32]),
    "tffn_session_set_bs1_path": (_i, [_vp, _i]),
    "tffn_session_capture_hidden": (_i, [_vp, _i]),
    "tffn_session_get_hidden": (_i, [_vp, _i, _vp, _i]),
    "tffn_prefill": (_i, [_vp, _vp, _vp, _i, _vp, _vp]),
    "tffn_forward": (_i, [_vp, _i, _vp, _i, _vp]),
    "tffn_decode_step": (_i, [_vp, _vp, _i, _vp, _vp]),
    "tffn_decode_run": (_i, [_vp, _i, _i, _vp]),
    "tffn_session_profile": (_i, [_vp, _i]),
    "tffn_session_profile_read": (_i, [_vp, _vp, _vp, _i]),
    "tffn_profile_class_name": (_cp, [_i]),
    "tffn_session_timeline": (_i, [_vp, _i, _vp, _i, _i, _vp, _i]),
    "tffn_session_status": (_i, [_vp]),
    "tffn_session_launch_count": (ctypes.c_uint64, [_vp]),
    "tffn_session_stream": (_vp, [_vp]),
    "tffn_op_gemm": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _i]),
    "tffn_op_gemm_trace": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _i]),
    "tffn_op_swiglu_bs1": (_i, [_i, _vp, _vp, _vp, _vp, _f, _f, _i, _i, _vp]),
    "tffn_op_swiglu_bs1_trace": (_i, [_i, _vp, _vp, _vp, _vp, _f, _f, _i, _i, _vp, _vp, _i]),
    "tffn_op_swiglu_bs1_noalloc": (_i, [_i, _vp, _vp, _vp, _vp, _f, _f, _i, _i, _vp]),
    "tffn_op_wait_selftest": (_i, [_i]),
    "tffn_op_tp_wait_selftest": (_i, [_i, _i]),
}
for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(_L, _name)
    _fn.restype = _res
    _fn.argtypes = _args
DECLARED_SYMBOLS = sorted(_SIGS)


def _check(rc: int) -> int:
    if rc < 0:
        raise TffnError(rc, (_L.tffn_last_error() or b"").decode("utf-8", "replace"))
    return rc


def _ptr(a):
    return None if a is None else a.ctypes.data


def device_count() -> int:
    return _L.tffn_device_count()


def qwen_config_from_json(model_dir: str) -> Config:
    """inference/src/model/qwen.cu:21-63"""
    c = Config()
    _check(_L.tffn_config_read(model_dir.encode(), ctypes.byref(c)))
    return c


def expert_probe(path: str):
    v = [ctypes.c_uint32() for _ in range(4)]
    _check(_L.tffn_expert_probe(path.encode(), *[ctypes.byref(x) for x in v]))
    return dict(version=v[0].value, num_layers=v[1].value, hidden=v[2].value, intermediate=v[3].value)


def checkpoint_save(path: str, mats: list[np.ndarray], num_layers: int, hidden: int, intermediate: int):
    """Writes the trainer's expert format (trainer/src/io/checkpoint.cpp:15-52); mats[l*3+m] fp32."""
    keep = [np.ascontiguousarray(m, dtype=np.float32).reshape(-1) for m in mats]
    assert len(keep) == num_layers * 3 and all(k.size == hidden * intermediate for k in keep)
    arr = (_vp * len(keep))(*[k.ctypes.data for k in keep])
    _check(_L.tffn_expert_write(path.encode(), num_layers, hidden, intermediate, arr))


def safetensors_probe(model_dir: str, name: str | None = None):
    ns, nt, nb = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_uint64()
    dt = ctypes.create_string_buffer(8)
    _check(_L.tffn_safetensors_probe(model_dir.encode(), name.encode() if name else None, ctypes.byref(ns),
                                     ctypes.byref(nt), dt, ctypes.byref(nb)))
    return dict(num_shards=ns.value, num_tensors=nt.value, dtype=dt.value.decode(), nbytes=nb.value)


class Tokenizer:
    """io::Tokenizer (inference/include/io/tokenizer.h:9-24)"""

    def __init__(self, model_dir: str):
        self._h = _vp()
        _check(_L.tffn_tokenizer_load(model_dir.encode(), ctypes.byref(self._h)))
        e, b, p = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_uint32()
        _check(_L.tffn_tokenizer_special(self._h, ctypes.byref(e), ctypes.byref(b), ctypes.byref(p)))
        self.eos_id, self.bos_id, self.pad_id = e.value, b.value, p.value

    def __del__(self):
        if getattr(self, "_h", None):
            _L.tffn_tokenizer_free(self._h)
            self._h = None

    def encode(self, text: str) -> list[int]:
        raw = text.encode("utf-8")
        n = _check(_L.tffn_tokenizer_encode(self._h, raw, None, 0))
        ids = np.zeros(max(n, 1), dtype=np.uint32)
        _check(_L.tffn_tokenizer_encode(self._h, raw, ids.ctypes.data, n))
        return [int(x) for x in ids[:n]]

    def decode(self, ids) -> str:
        a = np.ascontiguousarray(ids, dtype=np.uint32)
        n = _check(_L.tffn_tokenizer_decode(self._h, a.ctypes.data, a.size, None, 0))
        buf = ctypes.create_string_buffer(n + 1)
        _check(_L.tffn_tokenizer_decode(self._h, a.ctypes.data, a.size, buf, n + 1))
        return buf.raw[:n].decode("utf-8", "replace")

    def encode_bpe(self, text: str) -> list[int]:
        """the byte-level BPE tokenizer.json specifies (not the reference's space-dropping encoder)"""
        raw = text.encode("utf-8")
        n = _check(_L.tffn_tokenizer_encode_bpe(self._h, raw, None, 0))
        ids = np.zeros(max(n, 1), dtype=np.uint32)
        _check(_L.tffn_tokenizer_encode_bpe(self._h, raw, ids.ctypes.data, n))
        return [int(x) for x in ids[:n]]

    def decode_bpe(self, ids) -> str:
        a = np.ascontiguousarray(ids, dtype=np.uint32)
        n = _check(_L.tffn_tokenizer_decode_bpe(self._h, a.ctypes.data, a.size, None, 0))
        buf = ctypes.create_string_buffer(n + 1)
        _check(_L.tffn_tokenizer_decode_bpe(self._h, a.ctypes.data, a.size, buf, n + 1))
        return buf.raw[:n].decode("utf-8", "replace")

    def get_id(self, token: str) -> int:
        v = ctypes.c_uint32()
        _check(_L.tffn_tokenizer_token_id(self._h, token.encode(), ctypes.byref(v)))
        return v.value


class ExpertModel:
    """model::ExpertModel (inference/include/model/expert.h:13-27): device weights + output_scale."""

    def __init__(self, handle, model):
        self._h = handle
        self._model = model

    @property
    def output_scale(self) -> float:
        return _L.tffn_expert_get_scale(self._h)

    @output_scale.setter
    def output_scale(self, v: float):
        _check(_L.tffn_expert_set_scale(self._h, v))

    def expert_forward(self, x_norm_ptr: int, out_delta_ptr: int, batch_tokens: int, stream: int = 0):
        """expert_forward of the trainer (trainer/src/model/ffn_expert.cu:151-175): DEVICE pointers to
        bf16 [layers, batch_tokens, hidden] in and fp32 [layers, batch_tokens, hidden] out"""
        _check(_L.tffn_expert_forward(self._h, ctypes.c_void_p(x_norm_ptr), ctypes.c_void_p(out_delta_ptr), batch_tokens,
                                      ctypes.c_void_p(stream)))

    def free(self):
        if self._h:
            _L.tffn_expert_free(self._h)
            self._h = None

    def __del__(self):
        if _L is not None:  # module globals are gone at interpreter shutdown
            self.free()


class QwenModel:
    """model::QwenModel (inference/include/model/qwen.h:59-99) split into immutable weights (this
    object) and sessions that own the KV cache."""

    def __init__(self, handle):
        self._h = handle
        self.cfg = Config()
        _check(_L.tffn_model_config(self._h, ctypes.byref(self.cfg)))

    def weight_bytes(self, with_expert: bool) -> int:
        return int(_L.tffn_model_weight_bytes(self._h, int(with_expert)))

    def free(self):
        if self._h:
            _L.tffn_model_free(self._h)
            self._h = None

    def __del__(self):
        if _L is not None:  # module globals are gone at interpreter shutdown
            self.free()


def qwen_load(model_dir: str, device: int = 0, tp_rank: int = 0, tp_size: int = 1) -> QwenModel:
    """qwen_load without the KV cache (inference/src/model/qwen.cu:80-132); with tp_size > 1 this
    process loads only the slices of tensor-parallel rank tp_rank"""
    h = _vp()
    _check(_L.tffn_model_load(model_dir.encode(), device, tp_rank, tp_size, ctypes.byref(h)))
    return QwenModel(h)


def tp_unique_id() -> bytes:
    """the 128-byte id rank 0 hands to the other ranks of a tensor-parallel group"""
    buf = ctypes.create_string_buffer(128)
    _check(_L.tffn_tp_unique_id(buf))
    return buf.raw


class TpGroup:
    """NCCL communicator of a tensor-parallel group (one process per GPU); creation is collective"""

    def __init__(self, unique_id: bytes, tp_rank: int, tp_size: int, device: int):
        assert len(unique_id) == 128
        self.rank, self.size = tp_rank, tp_size
        self._h = _vp()
        _check(_L.tffn_tp_create(unique_id, tp_rank, tp_size, device, ctypes.byref(self._h)))

    def free(self):
        if getattr(self, "_h", None):
            _L.tffn_tp_free(self._h)
            self._h = None

    def __del__(self):
        if _L is not None:
            self.free()


def tp_rendezvous(directory: str, tp_rank: int, tp_size: int, timeout_s: float = 60.0) -> bytes:
    """File-based meeting point of a tensor-parallel group on one machine: rank 0 publishes the NCCL id,
    every rank signs in and waits until all tp_size ranks have. A rank that never arrives makes the
    others give up after timeout_s with TffnError(-6) instead of entering a collective that could not
    complete. Returns the 128-byte id for TpGroup."""
    import time
    os.makedirs(directory, exist_ok=True)
    idf = os.path.join(directory, "nccl_id")
    if tp_rank == 0:
        tmp = idf + ".tmp"
        with open(tmp, "wb") as f:
            f.write(tp_unique_id())
        os.replace(tmp, idf)
    with open(os.path.join(directory, f"rank{tp_rank}.here"), "w") as f:
        f.write("1")
    t_end = time.monotonic() + timeout_s
    while True:
        missing = [r for r in range(tp_size) if not os.path.exists(os.path.join(directory, f"rank{r}.here"))]
        if not missing and os.path.exists(idf):
            with open(idf, "rb") as f:
                return f.read()
        if time.monotonic() > t_end:
            raise TffnError(-6, f"tensor-parallel rendezvous timed out after {timeout_s:.0f} s: ranks {missing} of {tp_size} never arrived")
        time.sleep(0.02)


def tp_partition(cfg: Config, tp_rank: int, tp_size: int) -> dict:
    """what rank tp_rank of tp_size owns (host-only arithmetic): heads, intermediate rows, LM-head rows"""
    out = (ctypes.c_int32 * 8)()
    _check(_L.tffn_tp_partition(ctypes.byref(cfg), tp_rank, tp_size, out))
    keys = ("q_head0", "n_q_heads", "kv_head0", "n_kv_heads", "i0", "n_i", "v0", "n_v")
    return dict(zip(keys, [int(v) for v in out]))


def checkpoint_load(path: str, model: QwenModel, output_scale: float = kExpertOutputScale) -> ExpertModel:
    """expert_alloc + checkpoint_load (inference/src/model/expert.cu:9-31, src/io/checkpoint.cpp:11-65)"""
    h = _vp()
    _check(_L.tffn_expert_load(model._h, path.encode(), output_scale, ctypes.byref(h)))
    return ExpertModel(h, model)


class Session:
    """KV cache + scratch (the second half of qwen_load, inference/src/model/qwen.cu:134-171), paged."""

    def __init__(self, model: QwenModel, expert: ExpertModel | None = None, max_batch: int = 1, max_seq: int = 2048,
                 stream: int | None = None, tp: "TpGroup | None" = None):
        self.model, self.expert, self.tp = model, expert, tp
        self.max_batch, self.max_seq = max_batch, max_seq
        self.V = model.cfg.vocab_size
        self._h = _vp()
        _check(_L.tffn_session_create_tp(model._h, expert._h if expert else None, max_batch, max_seq, stream,
                                         tp._h if tp else None, ctypes.byref(self._h)))

    def free(self):
        if getattr(self, "_h", None):
            _L.tffn_session_free(self._h)
            self._h = None

    def __del__(self):
        if _L is not None:  # module globals are gone at interpreter shutdown
            self.free()

    def qwen_reset(self, slot: int = -1):
        """qwen_reset (inference/src/model/qwen.cu:174)"""
        _check(_L.tffn_session_reset(self._h, slot))

    def seq_len(self, slot: int = 0) -> int:
        return _check(_L.tffn_session_seq_len(self._h, slot))

    def set_launch_mode(self, mode: int):
        _check(_L.tffn_session_set_launch_mode(self._h, mode))

    def set_tp_fused(self, on: bool):
        """tensor parallel: False sends every all-reduce through NCCL (all ranks alike)"""
        _check(_L.tffn_session_set_tp_fused(self._h, 1 if on else 0))

    def set_ablation(self, mask: int):
        """timing aid: skip the kernel classes whose bit is set (results become meaningless)"""
        _check(_L.tffn_session_set_ablation(self._h, mask))

    def set_sampling(self, temperature: float, seed: int = 42):
        """temperature sampling on the device as sample() (inference/src/main.cpp:52-63); <= 0: greedy"""
        _check(_L.tffn_session_set_sampling(self._h, float(temperature), int(seed)))

    def set_bs1_path(self, on: bool):
        _check(_L.tffn_session_set_bs1_path(self._h, int(on)))

    def capture_hidden(self, max_rows: int):
        _check(_L.tffn_session_capture_hidden(self._h, max_rows))

    def get_hidden(self, layer: int, rows: int) -> np.ndarray:
        out = np.zeros((rows, self.model.cfg.hidden_size), dtype=np.uint16)
        n = _check(_L.tffn_session_get_hidden(self._h, layer, out.ctypes.data, rows))
        return out[:n]

    def qwen_forward(self, tokens, slot: int = 0, want_logits: bool = True):
        """qwen_forward (inference/src/model/qwen.cu:291-458): append T tokens, fp32 logits [T, V]."""
        tok = np.ascontiguousarray(tokens, dtype=np.int32)
        logits = np.empty((tok.size, self.V), dtype=np.float32) if want_logits else None
        _check(_L.tffn_forward(self._h, slot, tok.ctypes.data, tok.size, _ptr(logits)))
        return logits

    def prefill(self, prompts, want_logits: bool = False):
        """prompts: list of int sequences, one per slot starting at slot 0 -> (next tokens, last-row logits)."""
        lens = np.array([len(p) for p in prompts], dtype=np.int32)
        flat = np.ascontiguousarray(np.concatenate([np.asarray(p, dtype=np.int32) for p in prompts]))
        nxt = np.empty(len(prompts), dtype=np.int32)
        logits = np.empty((len(prompts), self.V), dtype=np.float32) if want_logits else None
        _check(_L.tffn_prefill(self._h, flat.ctypes.data, lens.ctypes.data, len(prompts), nxt.ctypes.data, _ptr(logits)))
        return nxt, logits

    def decode_step(self, tokens_in=None, n_seqs: int | None = None, want_logits: bool = False):
        if tokens_in is not None:
            tin = np.ascontiguousarray(tokens_in, dtype=np.int32)
            n_seqs = tin.size
        else:
            tin = None
        nxt = np.empty(n_seqs, dtype=np.int32)
        logits = np.empty((n_seqs, self.V), dtype=np.float32) if want_logits else None
        _check(_L.tffn_decode_step(self._h, _ptr(tin), n_seqs, nxt.ctypes.data, _ptr(logits)))
        return nxt, logits

    def decode_run(self, n_seqs: int, steps: int, want_tokens: bool = True):
        out = np.empty((steps, n_seqs), dtype=np.int32) if want_tokens else None
        _check(_L.tffn_decode_run(self._h, n_seqs, steps, _ptr(out)))
        return out

    def profile(self, on: bool):
        _check(_L.tffn_session_profile(self._h, int(on)))

    def profile_read(self) -> dict:
        """kernel class -> (device ms, launches) accumulated since profile(True)"""
        ms = np.zeros(64, dtype=np.float32)
        n = np.zeros(64, dtype=np.int32)
        k = _check(_L.tffn_session_profile_read(self._h, ms.ctypes.data, n.ctypes.data, 64))
        return {_L.tffn_profile_class_name(i).decode(): (float(ms[i]), int(n[i])) for i in range(k) if n[i] > 0}

    def timeline(self, n_seqs: int, max_launches: int = 1024, trace_launch: int = -1, trace_ctas: int = 0):
        """three batched decode steps; timeline of the last: (class names, uint64 [launches, 6] =
        min/max over CTAs of entry, grid-wait return, exit in globaltimer ns[, uint64 [trace_ctas, 64]
        per-CTA phase timestamps of GEMM launch number trace_launch])"""
        out = np.zeros((max_launches, 7), dtype=np.uint64)
        tr = np.zeros((max(trace_ctas, 1), 64), dtype=np.uint64)
        n = _check(_L.tffn_session_timeline(self._h, n_seqs, out.ctypes.data, max_launches, trace_launch,
                                            tr.ctypes.data if trace_ctas > 0 else None, trace_ctas))
        names = [_L.tffn_profile_class_name(int(c)).decode() for c in out[:n, 0]]
        if trace_ctas > 0:
            return names, out[:n, 1:], tr
        return names, out[:n, 1:]

    def status(self) -> int:
        return _check(_L.tffn_session_status(self._h))

    def launch_count(self) -> int:
        return int(_L.tffn_session_launch_count(self._h))

    def stream(self) -> int:
        return int(_L.tffn_session_stream(self._h) or 0)


def op_gemm(X: np.ndarray, W: np.ndarray, splits: int = 0, device: int = 0) -> np.ndarray:
    """X [T,K], W [N,K] as bf16 bit patterns (uint16) -> fp32 [T,N] on the tensor-core GEMM."""
    X = np.ascontiguousarray(X, dtype=np.uint16)
    W = np.ascontiguousarray(W, dtype=np.uint16)
    T, K = X.shape
    N = W.shape[0]
    out = np.empty((T, N), dtype=np.float32)
    _check(_L.tffn_op_gemm(device, X.ctypes.data, W.ctypes.data, out.ctypes.data, T, N, K, splits))
    return out


def op_gemm_trace(X: np.ndarray, W: np.ndarray, splits: int = 0, max_ctas: int = 4096, device: int = 0):
    """op_gemm plus per-CTA phase timestamps: returns (out, trace uint64 [max_ctas, 64], zeros where unused)"""
    X = np.ascontiguousarray(X, dtype=np.uint16)
    W = np.ascontiguousarray(W, dtype=np.uint16)
    T, K = X.shape
    N = W.shape[0]
    out = np.empty((T, N), dtype=np.float32)
    trace = np.zeros((max_ctas, 64), dtype=np.uint64)
    _check(_L.tffn_op_gemm_trace(device, X.ctypes.data, W.ctypes.data, out.ctypes.data, T, N, K, splits, trace.ctypes.data,
                                 max_ctas))
    return out, trace


def pack_ffn(gate: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    """gate, up [I,H], down [H,I] (bf16 bits) -> records [I][3][H]: gate row, up row, down column"""
    return np.ascontiguousarray(np.stack([gate, up, down.T], axis=1))


def op_swiglu_bs1(h, norm_w, packed_base, packed_expert=None, expert_scale=0.1, eps=1e-6, device: int = 0):
    """fused batch-1 FFN kernel: bf16 bits in, new residual stream (bf16 bits) out"""
    h = np.ascontiguousarray(h, dtype=np.uint16)
    w = np.ascontiguousarray(norm_w, dtype=np.uint16)
    pb = np.ascontiguousarray(packed_base, dtype=np.uint16)
    pe = None if packed_expert is None else np.ascontiguousarray(packed_expert, dtype=np.uint16)
    I, _, H = pb.shape
    out = np.empty(H, dtype=np.uint16)
    _check(_L.tffn_op_swiglu_bs1(device, h.ctypes.data, w.ctypes.data, pb.ctypes.data, _ptr(pe), expert_scale, eps, H, I,
                                 out.ctypes.data))
    return out


def op_swiglu_bs1_trace(h, norm_w, packed_base, packed_expert=None, expert_scale=0.1, eps=1e-6, max_ctas=256, device: int = 0):
    """op_swiglu_bs1 plus per-CTA phase timestamps of a warm launch: (h_out, trace uint64 [max_ctas, 16])"""
    h = np.ascontiguousarray(h, dtype=np.uint16)
    w = np.ascontiguousarray(norm_w, dtype=np.uint16)
    pb = np.ascontiguousarray(packed_base, dtype=np.uint16)
    pe = None if packed_expert is None else np.ascontiguousarray(packed_expert, dtype=np.uint16)
    I, _, H = pb.shape
    out = np.empty(H, dtype=np.uint16)
    trace = np.zeros((max_ctas, 16), dtype=np.uint64)
    _check(_L.tffn_op_swiglu_bs1_trace(device, h.ctypes.data, w.ctypes.data, pb.ctypes.data, _ptr(pe), expert_scale, eps, H, I,
                                       out.ctypes.data, trace.ctypes.data, max_ctas))
    return out, trace


def op_swiglu_bs1_noalloc(h_io_ptr: int, norm_w_ptr: int, packed_base_ptr: int, packed_expert_ptr: int | None, H: int, I: int,
                          expert_scale=0.1, eps=1e-6, stream: int | None = None, device: int = 0):
    """The same kernel for callers that cannot allocate: every argument is a DEVICE address the
    caller already owns, h_io is updated in place, scratch comes from a fixed array in the library."""
    _check(_L.tffn_op_swiglu_bs1_noalloc(device, h_io_ptr, norm_w_ptr, packed_base_ptr, packed_expert_ptr, expert_scale, eps,
                                         H, I, stream))


def op_wait_selftest(device: int = 0) -> int:
    return _check(_L.tffn_op_wait_selftest(device))


def op_tp_wait_selftest(wait_ms: int = 200, device: int = 0) -> int:
    """tensor-parallel hand-shake with a peer that never signals: the device status after the bounded wait (7)"""
    return _check(_L.tffn_op_tp_wait_selftest(device, wait_ms))
