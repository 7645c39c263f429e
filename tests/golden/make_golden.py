"""Generates tests/golden/golden_steps.npz from the COMPILED, UNMODIFIED reference CPU build
(oracle/_ref/libref_cpu.so, built by `make -C oracle ref` where the reference checkout is).

Run from the repository root:   python tests/golden/make_golden.py

For every small shape in SHAPES it records, through the reference's own functions:
  * the teacher-forced token sequence and the raw logits of every step (forward() body,
    src/model.cpp:373-380, captured before sample() mutates them),
  * the K/V cache rows the steps wrote (src/model.cpp:171-176),
  * sample() results (src/model.cpp:256-303) on the last step's logits for several
    (temperature, penalty) settings, with r taken from srand(1234)'s rand() stream,
  * outputs of the primitive ops (src/ops.cpp) on seeded inputs,
so that the plain-C restatement and the CUDA path can be checked where the reference is absent.
The model weights are not stored: they are regenerated from the seed by lighterpp_b200.synth.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from lighterpp_b200 import synth  # noqa: E402
from oracle.oracle import Reference  # noqa: E402

SHAPES = ["tiny-f32", "tiny-gqa-f16", "tiny-tp8-f16"]
N_STEPS = 12
SAMPLE_SETTINGS = [(0.0, 1.0), (0.0, 1.3), (1.0, 1.0), (0.8, 1.1)]
N_DRAWS = 16


def main():
    R = Reference()
    out = {}
    for name in SHAPES:
        c, dt, tied, seed, T = synth.named(name)
        m = R.model(c, synth.as_f32(T))
        toks = synth.prompt_tokens(c.vocab_size, N_STEPS, seed)
        logits = np.stack([m.step_logits(int(t), p) for p, t in enumerate(toks)])
        k, v = m.kv_cache()
        out[f"{name}/tokens"] = toks
        out[f"{name}/logits"] = logits
        out[f"{name}/k"] = k[:, :, :N_STEPS].copy()
        out[f"{name}/v"] = v[:, :, :N_STEPS].copy()
        hist = np.concatenate([toks, toks[:3], [-1, c.vocab_size + 5]]).astype(np.int32)
        out[f"{name}/history"] = hist
        rs = R.rand_floats(1234, N_DRAWS)
        out[f"{name}/r"] = rs
        ids = np.zeros((len(SAMPLE_SETTINGS), N_DRAWS), dtype=np.int32)
        for si, (temp, pen) in enumerate(SAMPLE_SETTINGS):
            R.srand(1234)  # draw di of a T>0 setting consumes rs[di]; T=0 consumes nothing (model.cpp:272-292)
            for di in range(N_DRAWS):
                ids[si, di] = R.sample(logits[-1], temp, pen, hist)
        out[f"{name}/sample_ids"] = ids
        m.close()
    out["sample_settings"] = np.array(SAMPLE_SETTINGS, dtype=np.float32)

    # primitive ops on seeded inputs
    rng = np.random.default_rng(99)
    x = rng.standard_normal(96).astype(np.float32)
    w = rng.standard_normal((40, 96)).astype(np.float32)
    g = rng.standard_normal(96).astype(np.float32)
    out["ops/x"], out["ops/w"], out["ops/g"] = x, w, g
    out["ops/matmul"] = R.matmul(x, w)
    out["ops/rmsnorm"] = R.rmsnorm(x, g)
    q, kk = R.rope(x, x[:48], 7, 48, 10000.0)
    out["ops/rope_q"], out["ops/rope_k"] = q, kk
    q2, kk2 = R.rope(x, x[:32], 33000, 32, 500000.0)
    out["ops/rope_q_far"], out["ops/rope_k_far"] = q2, kk2
    out["ops/softmax"] = R.softmax(x)
    out["ops/swiglu"] = R.swiglu(x, g)
    path = os.path.join(ROOT, "tests", "golden", "golden_steps.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
