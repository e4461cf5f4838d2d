"""-m gpu: tensor-ffn-inference --bpe end to end. The prompt is tokenised by the byte-level BPE of the model
directory's tokenizer.json (here one trained with HF `tokenizers` in the Qwen2 layout, small enough for the test
model's vocabulary) and the generated ids are printed through the matching decoder."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu
tokenizers = pytest.importorskip("tokenizers")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cli_bpe_prompt_and_output(model_dirs, tmp_path):
    from test_bpe_cpu import CORPUS, QWEN2_PATTERN, SPECIALS
    from tokenizers import Regex, Tokenizer, decoders, models, normalizers, pre_tokenizers, trainers
    cli = os.path.join(ROOT, "tensor-ffn_b200", "tensor-ffn-inference")
    d, ep, cfg = model_dirs["mini05"]  # vocabulary 1000
    t = Tokenizer(models.BPE())
    t.normalizer = normalizers.NFC()
    t.pre_tokenizer = pre_tokenizers.Sequence([
        pre_tokenizers.Split(Regex(QWEN2_PATTERN), behavior="isolated", invert=False),
        pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False),
    ])
    t.decoder = decoders.ByteLevel()
    t.train_from_iterator(CORPUS, trainers.BpeTrainer(vocab_size=700, special_tokens=SPECIALS, show_progress=False,
                                                      initial_alphabet=pre_tokenizers.ByteLevel.alphabet()))
    md = tmp_path / "model"
    shutil.copytree(d, md, symlinks=True)
    os.remove(md / "tokenizer.json")
    t.save(str(md / "tokenizer.json"))
    prompt = "def add(a, b):\n    return a + b  # café"
    want = len(t.encode(prompt, add_special_tokens=False).ids)
    r = subprocess.run([cli, "--model", str(md), "--expert", ep, "--prompt", prompt, "--bpe", "--max-tokens", "8", "--ignore-eos",
                        "--max-seq", "128", "--device", "0"], capture_output=True)
    assert r.returncode == 0, r.stderr.decode("utf-8", "replace")
    out = r.stdout.decode("utf-8", "replace")
    assert f"Prompt ({want} tokens)" in out, out
    # without --bpe the reference's encoder drops the spaces and newlines: a different token count
    r2 = subprocess.run([cli, "--model", str(md), "--expert", ep, "--prompt", prompt, "--max-tokens", "1", "--ignore-eos", "--max-seq",
                         "128", "--device", "0"], capture_output=True)
    assert r2.returncode == 0 and f"Prompt ({want} tokens)" not in r2.stdout.decode("utf-8", "replace")
    assert "Generating:" in out
