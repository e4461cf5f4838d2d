"""Generates the golden fixtures of tests/golden/ from the UNMODIFIED reference.

Run on a machine with a GPU, after `make -C oracle ref` has compiled the reference's own
inference sources into oracle/_ref/ref_driver:

    python tests/golden/make_golden.py --out tests/golden

For each case it writes a seeded synthetic model (tensor-ffn_b200/synth.py, the shapes of
tests/conftest.py), feeds a seeded token stream to the reference (prompt in one qwen_forward
call, then teacher-forced single-token calls) and stores what the reference produced:
all-row prompt logits + one logits row per decode step, the greedy picks, and the residual
stream after every layer for the prompt. The model files are not stored: they are a pure
function of the seeds recorded in the fixture.
"""
import argparse
import os
import subprocess
import sys
import tempfile

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.join(ROOT, "tensor-ffn_b200"))
sys.path.insert(0, os.path.join(ROOT, "tests"))

P, N = 16, 6  # prompt tokens, teacher-forced decode tokens
MODEL_SEED, EXPERT_SEED, NORM_JITTER = 1234, 4321, 0.1


def main():
    import synth
    from conftest import SHAPES
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    ap.add_argument("--driver", default=os.path.join(ROOT, "oracle", "_ref", "ref_driver"))
    a = ap.parse_args()
    os.makedirs(a.out, exist_ok=True)
    for name, (shape, bias) in SHAPES.items():
        with tempfile.TemporaryDirectory() as tmp:
            d = os.path.join(tmp, name)
            cfg = synth.write_model(d, shape, seed=MODEL_SEED, qkv_bias=bias, norm_jitter=NORM_JITTER)
            ep = os.path.join(d, "expert.bin")
            synth.write_expert(ep, cfg, seed=EXPERT_SEED)
            V, H, L = cfg["vocab_size"], cfg["hidden_size"], cfg["num_hidden_layers"]
            toks = synth.prompts(1, P + N, 42, V)[0]
            tf = os.path.join(tmp, "tokens.i32")
            toks.tofile(tf)
            for expert in (False, True):
                pre = os.path.join(tmp, f"out_{int(expert)}")
                cmd = [a.driver, "--model", d, "--max-seq", "64", "--tokens", tf, "--prompt-len", str(P), "--new", str(N),
                       "--out", pre, "--teacher", "--all-logits", "--hidden"]
                if expert:
                    cmd += ["--expert", ep, "--expert-scale", "0.1"]
                subprocess.check_call(cmd)
                logits = np.fromfile(pre + ".logits.f32", dtype=np.float32).reshape(P + N, V)
                picks = np.fromfile(pre + ".tokens.i32", dtype=np.int32)
                hidden = np.fromfile(pre + ".hidden.bf16", dtype=np.uint16).reshape(L, P, H)
                np.savez_compressed(os.path.join(a.out, f"ref_{name}_{'expert' if expert else 'base'}.npz"),
                                    shape_name=name, tokens=toks, prompt_len=P, logits=logits, picks=picks, hidden=hidden,
                                    model_seed=MODEL_SEED, expert_seed=EXPERT_SEED, norm_jitter=NORM_JITTER,
                                    qkv_bias=bias, expert=expert, expert_scale=0.1)
                print("wrote", name, expert, logits.shape, flush=True)


if __name__ == "__main__":
    main()
