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

It also stores what the TRAINER's own expert_forward (trainer/src/model/ffn_expert.cu:151-175, through
oracle/_ref/ref_trainer_driver) returns for seeded training-shaped inputs [layers, batch_tokens, hidden] and
the seeded expert weights of two shapes: the fixtures trainer_expert_forward_*.npz pin the restatement
(oracle.expert_forward_ref) that tffn_expert_forward is checked against.
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
sys.path.insert(0, os.path.join(ROOT, "oracle"))

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
    trainer_driver = os.path.join(os.path.dirname(a.driver), "ref_trainer_driver")
    if os.path.exists(trainer_driver):
        trainer_expert_forward(a.out, trainer_driver)


def trainer_expert_forward(out_dir, driver):
    """fixtures of the trainer's expert_forward: x (bf16 bits), out (fp32), the seeds of the expert weights"""
    import synth
    from conftest import SHAPES
    for name, T in (("tiny", 37), ("mini05", 64)):
        shape, _ = SHAPES[name]
        cfg = synth.make_config(shape)
        H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
        with tempfile.TemporaryDirectory() as tmp:
            ep = os.path.join(tmp, "expert.bin")
            synth.write_expert(ep, cfg, seed=EXPERT_SEED)
            data = np.memmap(ep, dtype=np.float32, mode="r", offset=20, shape=(L, 3, I * H))
            w = synth.f32_to_bf16(np.ascontiguousarray(data).reshape(-1))  # RNE, as checkpoint_load casts
            x = synth.f32_to_bf16(np.random.default_rng([77, T]).standard_normal((L, T, H), dtype=np.float32))
            wf, xf, of = (os.path.join(tmp, n) for n in ("w.bf16", "x.bf16", "out.f32"))
            w.tofile(wf)
            x.tofile(xf)
            subprocess.check_call([driver, str(L), str(H), str(I), str(T), wf, xf, of])
            out = np.fromfile(of, dtype=np.float32).reshape(L, T, H)
        np.savez_compressed(os.path.join(out_dir, f"trainer_expert_forward_{name}.npz"), shape_name=name, x=x, out=out,
                            batch_tokens=T, expert_seed=EXPERT_SEED, scale=0.01)
        print("wrote trainer expert_forward", name, out.shape, float(np.abs(out).max()), flush=True)


if __name__ == "__main__":
    main()
