"""CPU tests of the C-ABI boundary: the library loads, exports every symbol the header declares,
and reports errors through status codes (no compute calls without a GPU)."""
import ctypes as C
import os
import re

import pytest

from lighterpp_b200 import engine as E, synth

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_symbols():
    text = open(os.path.join(ROOT, "include", "lpp_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(lpp_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = E.load_library()
    syms = _header_symbols()
    assert len(syms) >= 30
    missing = [s for s in syms if not hasattr(lib, s)]
    assert not missing, missing
    assert sorted(E.EXPORTS) == syms  # the Python binding list is in step with the header


def test_strerror_and_status_codes():
    lib = E.load_library()
    assert lib.lpp_strerror(0) == b"ok"
    for code in range(1, 8):
        assert lib.lpp_strerror(code) not in (b"ok", b"unknown status")
    assert lib.lpp_strerror(99) == b"unknown status"


def test_invalid_arguments_are_rejected_without_a_device():
    lib = E.load_library()
    h = C.c_void_p()
    assert lib.lpp_engine_create(None, None, C.byref(h)) == 1
    c, dt, tied, seed = synth.SHAPES["tiny-f32"]
    bad = E.Config(c.dim, c.hidden_dim, c.n_layers, 5, c.n_kv_heads, c.vocab_size, c.seq_len, c.rope_base, 0, 0, 0, 1, 0,
                   0, 0, 0)
    assert lib.lpp_engine_create(C.byref(bad), None, C.byref(h)) == 1  # dim % n_heads != 0
    assert b"n_heads" in lib.lpp_last_error()
    bad_tp = E.Config(c.dim, c.hidden_dim, c.n_layers, c.n_heads, c.n_kv_heads, c.vocab_size, c.seq_len, c.rope_base, 0,
                      0, 0, 3, 0, 0, 0, 0)
    assert lib.lpp_engine_create(C.byref(bad_tp), None, C.byref(h)) == 1  # tp 3 does not divide 2 kv heads
    assert lib.lpp_step(None, 0, 0, None, None, 0, 0.0, None) == 1
    assert lib.lpp_finalize(None) == 1
    assert lib.lpp_engine_destroy(None) == 0
    assert lib.lpp_op_gemv(None, None, None, 4, 4, 0, None) == 1


def test_engine_fails_loudly_without_gpu():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    c, dt, tied, seed = synth.SHAPES["tiny-f32"]
    with pytest.raises(E.LppError) as ei:
        E.Engine(c, dt, "f32")
    assert ei.value.status == 7  # LPP_ERR_NO_DEVICE: no silent CPU fallback


def test_product_code_does_not_touch_the_oracle():
    """Nothing under lighterpp_b200/ may import, load or execute oracle/."""
    pkg = os.path.join(ROOT, "lighterpp_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h", ".sh")):
                text = open(os.path.join(dirpath, f), errors="replace").read()
                for needle in ("import oracle", "from oracle", "oracle/", "oracle.oracle", "liblpp_oracle",
                               "libref_cpu"):
                    assert needle not in text, (os.path.join(dirpath, f), needle)


def test_library_is_the_product_build():
    """The timing-aid environment switches (kernel kinds left out, arithmetic skipped ...) exist only in builds
    made with -DLPP_TIMING_AIDS; the library that ships must not contain them."""
    with open(E.LIB_PATH, "rb") as f:
        blob = f.read()
    for name in (b"LPP_DEBUG_SKIP", b"LPP_DEBUG_GEMV", b"LPP_STAGE_KB", b"LPP_ATTN_CHUNK", b"LPP_ATTN_CUDA_CORES"):
        assert name not in blob, name
