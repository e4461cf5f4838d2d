"""CPU: the host side of the boundary — file formats, tokenizer, command line, C-ABI surface.
No compute call is made here (there is no GPU and no CPU fallback)."""
import json
import os
import re
import struct
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "tensor-ffn_b200", "tensor-ffn-inference")


def test_library_exports_every_declared_symbol():
    """every function include/*.h declares is exported by libtffn.so and bound by the Python mirror"""
    import tffn
    inc = os.path.join(ROOT, "include")
    header = "".join(open(os.path.join(inc, f)).read() for f in sorted(os.listdir(inc)) if f.endswith(".h"))
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = sorted(set(re.findall(r"\b(tffn_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) >= 40
    out = subprocess.check_output(["nm", "-D", "--defined-only", tffn.LIB_PATH], text=True)
    exported = set(re.findall(r" T (tffn_[a-z0-9_]+)", out))
    assert not [d for d in declared if d not in exported], "declared but not exported"
    assert sorted(tffn.DECLARED_SYMBOLS) == declared, "Python mirror and header disagree"
    assert tffn.device_count() >= 0 and tffn._L.tffn_version() >= 100


def test_no_gpu_means_loud_failure_not_fallback(model_dirs):
    import tffn
    if tffn.device_count() > 0:
        pytest.skip("a GPU is present")
    d, ep, cfg = model_dirs["tiny"]
    with pytest.raises(tffn.TffnError) as ei:
        tffn.qwen_load(d)
    assert ei.value.code == -5 and "CUDA" in ei.value.msg


def test_config_reader_defaults_and_eos_forms(tmp_path):
    """same keys/defaults as qwen_config_from_json; eos/bos as int or array (first element)"""
    import tffn
    d = tmp_path / "m"
    d.mkdir()
    (d / "config.json").write_text(json.dumps({"hidden_size": 1536, "num_attention_heads": 12, "num_key_value_heads": 2,
                                               "eos_token_id": [7, 9], "bos_token_id": 5, "head_dim": 999,
                                               "tie_word_embeddings": False, "rope_theta": 10000.0}))
    c = tffn.qwen_config_from_json(str(d))
    assert (c.hidden_size, c.num_heads, c.num_kv_heads, c.head_dim) == (1536, 12, 2, 128)  # head_dim key is ignored
    assert (c.intermediate_size, c.num_layers, c.vocab_size) == (4864, 24, 151936)  # reference defaults
    assert (c.eos_token_id, c.bos_token_id, c.tie_embeddings) == (7, 5, 0)
    assert abs(c.rope_theta - 10000.0) < 1e-3 and abs(c.rms_norm_eps - 1e-6) < 1e-12
    (d / "config.json").write_text("{}")
    c = tffn.qwen_config_from_json(str(d))
    assert (c.hidden_size, c.eos_token_id, c.bos_token_id, c.tie_embeddings) == (896, 151645, 151643, 1)
    (d / "config.json").write_text('{"hidden_size": 100, "num_attention_heads": 3}')
    with pytest.raises(tffn.TffnError):
        tffn.qwen_config_from_json(str(d))
    with pytest.raises(tffn.TffnError) as ei:
        tffn.qwen_config_from_json(str(tmp_path / "nope"))
    assert ei.value.code == -2


def test_safetensors_reader(tmp_path):
    import synth
    import tffn
    d = str(tmp_path / "sharded")
    cfg = synth.write_model(d, "tiny", shard_bytes=300_000)  # forces several shards
    info = tffn.safetensors_probe(d, "model.layers.1.mlp.down_proj.weight")
    assert info["num_shards"] > 1 and info["dtype"] == "BF16"
    assert info["nbytes"] == cfg["hidden_size"] * cfg["intermediate_size"] * 2
    assert info["num_tensors"] == len(synth.tensor_specs(cfg))
    with pytest.raises(tffn.TffnError) as ei:
        tffn.safetensors_probe(d, "model.layers.9.mlp.down_proj.weight")
    assert ei.value.code == -3 and "Missing tensor" in ei.value.msg
    # malformed files: short header, header length past the end, offsets out of range, unknown dtype
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "a.safetensors").write_bytes(b"\x01\x02")
    with pytest.raises(tffn.TffnError):
        tffn.safetensors_probe(str(bad))
    (bad / "a.safetensors").write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(tffn.TffnError):
        tffn.safetensors_probe(str(bad))
    for hdr in ({"x": {"dtype": "BF16", "shape": [4], "data_offsets": [0, 64]}},
                {"x": {"dtype": "Q4", "shape": [4], "data_offsets": [0, 8]}},
                {"x": {"dtype": "BF16", "shape": [5], "data_offsets": [0, 8]}}):
        hj = json.dumps(hdr).encode()
        (bad / "a.safetensors").write_bytes(struct.pack("<Q", len(hj)) + hj + b"\0" * 8)
        with pytest.raises(tffn.TffnError) as ei:
            tffn.safetensors_probe(str(bad))
        assert ei.value.code == -3
    empty = tmp_path / "empty"
    empty.mkdir()
    with pytest.raises(tffn.TffnError):
        tffn.safetensors_probe(str(empty))


def test_expert_bin_round_trip_and_errors(tmp_path):
    """writer == trainer's checkpoint_save format; reader checks magic and length; version is read, not checked"""
    import synth
    import tffn
    L, H, I = 2, 16, 24
    rng = np.random.default_rng(0)
    mats = [rng.standard_normal(H * I).astype(np.float32) for _ in range(L * 3)]
    p = str(tmp_path / "e.bin")
    tffn.checkpoint_save(p, mats, L, H, I)
    raw = open(p, "rb").read()
    assert struct.unpack("<5I", raw[:20]) == (0x45585054, 1, L, H, I)
    assert raw[20:] == b"".join(m.tobytes() for m in mats)  # bit-exact payload, gate/up/down per layer
    assert tffn.expert_probe(p) == dict(version=1, num_layers=L, hidden=H, intermediate=I)
    # the generator writes the same bytes for the same content
    cfg = dict(num_hidden_layers=L, hidden_size=H, intermediate_size=I)
    synth.write_expert(str(tmp_path / "g.bin"), cfg, seed=5)
    assert tffn.expert_probe(str(tmp_path / "g.bin"))["hidden"] == H
    synth.write_expert(str(tmp_path / "trunc.bin"), cfg, seed=5, truncate_bytes=4)
    with pytest.raises(tffn.TffnError) as ei:
        tffn.expert_probe(str(tmp_path / "trunc.bin"))
    assert ei.value.code == -3 and "truncated" in ei.value.msg
    synth.write_expert(str(tmp_path / "magic.bin"), cfg, seed=5, magic=0x12345678)
    with pytest.raises(tffn.TffnError) as ei:
        tffn.expert_probe(str(tmp_path / "magic.bin"))
    assert "Bad checkpoint magic: 0x12345678 (expected 0x45585054)" in ei.value.msg
    open(str(tmp_path / "v9.bin"), "wb").write(struct.pack("<5I", 0x45585054, 9, L, H, I) + raw[20:])
    assert tffn.expert_probe(str(tmp_path / "v9.bin"))["version"] == 9
    with pytest.raises(tffn.TffnError) as ei:
        tffn.expert_probe(str(tmp_path / "missing.bin"))
    assert ei.value.code == -2


def _ref_tokenizer(model_dir):
    """Python restatement of inference/src/io/tokenizer.cpp:16-153 used as the checker"""
    j = json.load(open(os.path.join(model_dir, "tokenizer.json")))
    t2i = dict(j["model"]["vocab"])
    i2t = {v: k for k, v in t2i.items()}
    merges, rank = [], {}
    for m in j["model"]["merges"]:
        a, b = m.split(" ", 1)
        if a in t2i and b in t2i:
            rank.setdefault((t2i[a], t2i[b]), len(merges))
            merges.append((t2i[a], t2i[b]))
    for at in j.get("added_tokens", []):
        t2i[at["content"]] = at["id"]
        i2t[at["id"]] = at["content"]

    def encode(text):
        ids = []
        for c in text.encode("utf-8"):
            s = bytes([c]).decode("latin-1") if c < 128 else None
            if s is not None and s in t2i:
                ids.append(t2i[s])
            elif "<0x%02X>" % c in t2i:
                ids.append(t2i["<0x%02X>" % c])
        changed = True
        while changed and len(ids) > 1:
            changed = False
            best, pos = None, 0
            for i in range(len(ids) - 1):
                r = rank.get((ids[i], ids[i + 1]))
                if r is not None and (best is None or r < best):
                    best, pos = r, i
            if best is not None:
                merged = i2t[merges[best][0]] + i2t[merges[best][1]]
                if merged in t2i:
                    ids[pos:pos + 2] = [t2i[merged]]
                    changed = True
        return ids

    def decode(ids):
        return "".join(i2t.get(i, "") for i in ids).replace("Ġ", " ")
    return encode, decode


def test_tokenizer_matches_reference_behaviour(model_dirs):
    import tffn
    d, ep, cfg = model_dirs["tiny"]
    tok = tffn.Tokenizer(d)
    enc, dec = _ref_tokenizer(d)
    for text in ["the rain in then", "func main() { return there; }", "a b\nc", "", "~~~", "iné"]:
        ids = tok.encode(text)
        assert ids == enc(text), text
        assert tok.decode(ids) == dec(ids)
    assert "the" in tok.decode(tok.encode("the")) and len(tok.encode("the")) == 1  # merges t+h, th+e applied
    assert tok.encode("a b") == tok.encode("ab")  # like the reference: a space has no vocab entry and is dropped
    gc = json.load(open(os.path.join(d, "generation_config.json")))
    assert tok.eos_id == gc["eos_token_id"][0] and tok.bos_id == gc["bos_token_id"] and tok.pad_id == tok.bos_id
    assert tok.get_id("<|im_start|>") > 0 and tok.get_id("<|nope|>") == 0
    with pytest.raises(tffn.TffnError):
        tffn.Tokenizer(os.path.join(d, "missing"))


def test_cli_flags_and_errors(model_dirs):
    """usage text and exit codes of inference/src/main.cpp:17-31,76-95; the model load fails loudly without a GPU"""
    import tffn
    d, ep, cfg = model_dirs["tiny"]
    r = subprocess.run([CLI], capture_output=True, text=True)
    assert r.returncode == 1 and "--model        <dir>" in r.stderr and "--max-seq      <N>" in r.stderr
    r = subprocess.run([CLI, "--model", d], capture_output=True, text=True)
    assert r.returncode == 1 and "--model and --prompt are required" in r.stderr
    # a flag in the last position has no value: like the reference it is not seen
    r = subprocess.run([CLI, "--model", d, "--prompt"], capture_output=True, text=True)
    assert r.returncode == 1 and "required" in r.stderr
    r = subprocess.run([CLI, "inference", "--model", os.path.join(d, "missing"), "--prompt", "x"], capture_output=True, text=True)
    assert r.returncode == 1 and "tokenizer.json" in r.stderr
    if tffn.device_count() == 0:
        r = subprocess.run([CLI, "--model", d, "--prompt", "the"], capture_output=True, text=True)
        assert r.returncode == 1 and "CUDA" in r.stderr and "Generating" not in r.stdout
