"""Drop-in proof on the GPU: the reference's OWN host code, compiled unmodified with -DUSE_CUDA and linked against
liblpp_b200.so through the C++ shim (lighterpp_b200/csrc/shim), runs on this engine.

* oracle/_ref/runtests_b200      = src/runtests.cpp (six CPU known-answer tests + nine CUDA-vs-CPU operator tests)
* oracle/_ref/lighterpp_b200_cli = src/main.cpp + src/loader.cpp + src/gguf.cpp + src/tokenizer.cpp: the reference CLI

Both are built by `make -C oracle dropin` where the reference checkout is present and travel as binaries."""
import os
import re
import subprocess

import numpy as np
import pytest

from lighterpp_b200 import formats, synth

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUNTESTS = os.path.join(ROOT, "oracle", "_ref", "runtests_b200")
CLI = os.path.join(ROOT, "oracle", "_ref", "lighterpp_b200_cli")


def _need(path):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    if not os.path.exists(path):
        pytest.skip(f"{os.path.basename(path)} not built (needs the reference checkout at build time)")


def test_reference_runtests_pass_on_the_shim():
    _need(RUNTESTS)
    r = subprocess.run([RUNTESTS], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert "ALL TESTS PASSED" in r.stdout
    assert r.stdout.count("PASSED") >= 16  # 6 KATs (7 checks) + 9 CUDA operator tests


def test_reference_cli_generates_the_engine_tokens(tmp_path):
    """`Lighter++ model.gguf -t 0`: main.cpp's own load / prefill / generate loop (src/main.cpp:115-232) on the engine,
    compared token by token with the same loop driven from Python."""
    _need(CLI)
    from lighterpp_b200 import engine as E
    name = "mini-long-f16"
    c, dt, tied, seed, T = synth.named(name)
    path = str(tmp_path / "m.gguf")
    formats.write_gguf(path, c, T)
    r = subprocess.run([CLI, path, "-t", "0"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    body = r.stdout.split("--- Running Inference ---")[1].split("--- Statistics ---")[0]
    cli_tokens = [int(t) for t in re.findall(r"t(\d+)", body)]
    # the same loop in Python: BOS = 1, greedy, penalty 1.05 over a 64-entry history (src/main.cpp:149-223)
    eng = E.Engine(c, dt, "f16")
    eng.load_weights(T)
    tok, hist, want = 1, [1], [1]
    for pos in range(200):
        tok = eng.forward(tok, pos, 0.0, 1.05, hist, 0.0)
        hist = (hist + [tok])[-64:]
        if tok in (2, 128001, 128009):
            break
        want.append(tok)
    eng.close()
    assert len(cli_tokens) >= 100
    assert cli_tokens == want[:len(cli_tokens)] and len(cli_tokens) == len(want)


def _write_tokenizer_bin(path, vocab_size):
    """The llama2.c tokenizer file src/tokenizer.cpp:16-56 reads: max token length, then (score, length, bytes) per
    token; token i is the string "t<i>" so that the CLI's output can be read back as ids."""
    import struct
    with open(path, "wb") as f:
        f.write(struct.pack("<i", 8))
        for i in range(vocab_size):
            s = f"t{i}".encode()
            f.write(struct.pack("<fi", 0.0, len(s)) + s)


def test_reference_cli_on_a_llama2c_bin(tmp_path):
    """`Lighter++ model.bin tokenizer.bin -t 0`: the llama2.c checkpoint path of the reference's loader
    (src/loader.cpp:18-172: mmap, FP32 tensors, tied classifier, device upload) feeding the engine through the shim."""
    _need(CLI)
    from lighterpp_b200 import engine as E
    from lighterpp_b200.formats import ModelConfig
    c = ModelConfig(96, 256, 2, 2, 2, 320, 256, 10000.0)
    T = synth.gen_model(c, 21, "f32", True)
    path, tok_path = str(tmp_path / "m.bin"), str(tmp_path / "tok.bin")
    formats.write_llama2c_bin(path, c, T)
    _write_tokenizer_bin(tok_path, c.vocab_size)
    r = subprocess.run([CLI, path, tok_path, "-t", "0"], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    body = r.stdout.split("--- Running Inference ---")[1].split("--- Statistics ---")[0]
    cli_tokens = [int(t) for t in re.findall(r"t(\d+)", body)]
    eng = E.Engine(c, "f32", "f16")  # the shim keeps the reference GPU path's FP16 cache
    eng.load_weights(T)
    tok, hist, want = 1, [1], [1]
    for pos in range(200):
        tok = eng.forward(tok, pos, 0.0, 1.05, hist, 0.0)
        hist = (hist + [tok])[-64:]
        if tok in (2, 128001, 128009):
            break
        want.append(tok)
    eng.close()
    assert len(cli_tokens) >= 100
    assert cli_tokens == want[:len(cli_tokens)] and len(cli_tokens) == len(want)
