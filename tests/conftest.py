import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "tensor-ffn_b200"), os.path.join(ROOT, "oracle"), ROOT):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def _have_gpu() -> bool:
    try:
        import tffn
        return tffn.device_count() > 0
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _have_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


SHAPES = {
    # name -> (synth shape dict, qkv_bias)
    "tiny": (dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                  intermediate_size=512, vocab_size=1024, tie_word_embeddings=True), True),
    "tiny128": (dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1,
                     intermediate_size=384, vocab_size=640, tie_word_embeddings=False), False),
    # the 0.5B head geometry (7 query heads per kv head, hidden not a multiple of 128) at small size
    "mini05": (dict(hidden_size=448, num_hidden_layers=3, num_attention_heads=7, num_key_value_heads=1,
                    intermediate_size=608, vocab_size=1000, tie_word_embeddings=True), True),
    # the same head geometry with an intermediate size that is a multiple of 256
    "mini_s": (dict(hidden_size=448, num_hidden_layers=3, num_attention_heads=7, num_key_value_heads=1,
                    intermediate_size=768, vocab_size=1000, tie_word_embeddings=True), True),
    # the 7B head geometry (7 query heads per kv head, more than one kv head) for tensor-parallel splits of 2, 4 and 8
    "mini7": (dict(hidden_size=896, num_hidden_layers=2, num_attention_heads=14, num_key_value_heads=2,
                   intermediate_size=1024, vocab_size=2048, tie_word_embeddings=False), True),
}


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """name -> (model dir, expert path, cfg); written once per test session."""
    import synth
    out = {}
    base = tmp_path_factory.mktemp("models")
    for name, (shape, bias) in SHAPES.items():
        d = str(base / name)
        cfg = synth.write_model(d, shape, seed=1234, qkv_bias=bias, norm_jitter=0.1)
        ep = os.path.join(d, "expert.bin")
        synth.write_expert(ep, cfg, seed=4321)
        out[name] = (d, ep, cfg)
    return out
