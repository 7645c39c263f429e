"""ctypes front-end for the two CPU checkers.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

* ``Oracle``    -- the plain-C restatement ``liblpp_oracle.so`` (oracle/lpp_oracle.c).
* ``Reference`` -- the unmodified reference CPU build ``_ref/libref_cpu.so`` (oracle/Makefile
  target ``ref``; only available where it was built from the reference checkout).

Only tests/, ``__graft_entry__.smoke()`` and bench.py's cpu_baseline / reference arm import this.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from typing import Dict, Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liblpp_oracle.so")
REF_SO = os.path.join(HERE, "_ref", "libref_cpu.so")


def reference_checkout() -> Optional[str]:
    """Where the Lighter++ sources lie: $LPP_REFERENCE, else a directory named ``reference`` beside this
    repository; None when neither holds a ``src`` folder."""
    for cand in (os.environ.get("LPP_REFERENCE"), os.path.join(HERE, "..", "..", "reference")):
        if cand and os.path.isdir(os.path.join(cand, "src")):
            return os.path.abspath(cand)
    return None


_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)
_WEIGHT_ORDER = ["tok_emb", "rms_att", "wq", "wk", "wv", "wo", "rms_ffn", "w1", "w2", "w3", "rms_final", "w_cls"]


def build(ref: bool = True) -> None:
    """Compile the restatement, and the reference CPU build when its checkout is present."""
    subprocess.run(["make", "-s", "-C", HERE, "oracle"], check=True)
    checkout = reference_checkout() if ref else None
    if checkout:
        subprocess.run(["make", "-s", "-C", HERE, "ref", f"REF={checkout}"], check=True)
        # the reference's own main.cpp / runtests.cpp linked against the CUDA library through the C++ shim
        if os.path.exists(os.path.join(HERE, "..", "lighterpp_b200", "liblpp_b200.so")):
            subprocess.run(["make", "-s", "-C", HERE, "dropin", f"REF={checkout}"], check=True)


def have_reference() -> bool:
    return os.path.exists(REF_SO)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a: Optional[np.ndarray]):
    return a.ctypes.data_as(_fp) if a is not None else None


class _ModelBase:
    """Shared driver logic; subclasses bind the prefix-specific symbols."""

    def __init__(self, lib, prefix: str, cfg, weights: Dict[str, np.ndarray], keep_f16: bool = False):
        self.lib, self.p, self.cfg = lib, prefix, cfg
        if keep_f16:
            # binary16 matrices stay binary16 (widened exactly inside the C code): half the host memory of FP32
            # copies, which is what makes the 8B shape fit.  Norm weights are FP32 as everywhere.
            self._w = {k: (_f32(v) if k.startswith("rms") else np.ascontiguousarray(v, dtype=np.float16))
                       for k, v in weights.items() if k in _WEIGHT_ORDER}
            create = getattr(lib, prefix + "create_f16")
        else:
            # keep FP32 copies alive for the lifetime of the C model
            self._w = {k: _f32(weights[k]) for k in _WEIGHT_ORDER if k in weights}
            create = getattr(lib, prefix + "create")
        create.restype = C.c_void_p
        create.argtypes = [C.c_int] * 7 + [C.c_float] + [C.c_void_p] * 12
        ptrs = [self._w[k].ctypes.data if k in self._w else None for k in _WEIGHT_ORDER]
        self.h = create(cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.vocab_size,
                        cfg.seq_len, cfg.rope_base, *ptrs)
        self._bind()

    def _bind(self):
        lib, p = self.lib, self.p
        f = getattr(lib, p + "step_logits")
        f.restype, f.argtypes = None, [C.c_void_p, C.c_int, C.c_int, _fp]
        self._step = f
        for n in ("key_cache", "value_cache"):
            g = getattr(lib, p + n)
            g.restype, g.argtypes = _fp, [C.c_void_p]
        fr = getattr(lib, p + "free")
        fr.restype, fr.argtypes = None, [C.c_void_p]

    def step_logits(self, token: int, pos: int) -> np.ndarray:
        out = np.empty(self.cfg.vocab_size, dtype=np.float32)
        self._step(self.h, int(token), int(pos), _ptr(out))
        return out

    def kv_cache(self):
        """(key, value) views shaped [L][KVH][seq_len][head_size] (src/model.cpp:173)."""
        c = self.cfg
        shape = (c.n_layers, c.n_kv_heads, c.seq_len, c.head_size)
        n = int(np.prod(shape))
        k = np.ctypeslib.as_array(getattr(self.lib, self.p + "key_cache")(self.h), shape=(n,)).reshape(shape)
        v = np.ctypeslib.as_array(getattr(self.lib, self.p + "value_cache")(self.h), shape=(n,)).reshape(shape)
        return k, v

    def close(self):
        if self.h:
            getattr(self.lib, self.p + "free")(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class Oracle:
    """Stateless ops of the restatement plus a model factory."""

    def __init__(self):
        if not os.path.exists(ORACLE_SO):
            build(ref=False)
        self.lib = lib = C.CDLL(ORACLE_SO)
        lib.oracle_matmul.argtypes = [_fp, _fp, _fp, C.c_int, C.c_int]
        lib.oracle_rmsnorm.argtypes = [_fp, _fp, _fp, C.c_int]
        lib.oracle_rope.argtypes = [_fp, _fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
        lib.oracle_rope_cos_sin.argtypes = [C.c_int, C.c_int, C.c_int, C.c_float, _fp, _fp]
        lib.oracle_softmax.argtypes = [_fp, C.c_int]
        lib.oracle_swiglu.argtypes = [_fp, _fp, _fp, C.c_int]
        lib.oracle_kv_index.restype = C.c_int64
        lib.oracle_kv_index.argtypes = [C.c_int] * 7
        lib.oracle_sample.restype = C.c_int
        lib.oracle_sample.argtypes = [_fp, C.c_int, C.c_float, C.c_float, _ip, C.c_int, C.c_float]
        lib.oracle_sample_exp_repro.restype = C.c_int
        lib.oracle_sample_exp_repro.argtypes = [_fp, C.c_int, C.c_float, C.c_float, _ip, C.c_int, C.c_float]
        lib.oracle_srand.argtypes = [C.c_uint]
        lib.oracle_rand_floats.argtypes = [_fp, C.c_int]

    def model(self, cfg, weights, keep_f16: bool = False) -> _ModelBase:
        """keep_f16: hand binary16 matrices to the C code as they are (exact widening on use) instead of
        making FP32 copies; results are bit-identical, host memory is halved."""
        return _ModelBase(self.lib, "oracle_", cfg, weights, keep_f16)

    def matmul(self, x, w):
        x, w = _f32(x), _f32(w)
        out = np.empty(w.shape[0], dtype=np.float32)
        self.lib.oracle_matmul(_ptr(out), _ptr(x), _ptr(w), w.shape[0], w.shape[1])
        return out

    def rmsnorm(self, x, weight):
        x, weight = _f32(x), _f32(weight)
        out = np.empty_like(x)
        self.lib.oracle_rmsnorm(_ptr(out), _ptr(x), _ptr(weight), x.size)
        return out

    def rope(self, q, k, pos, head_size, rope_base):
        q, k = _f32(q).copy(), _f32(k).copy()
        self.lib.oracle_rope(_ptr(q), _ptr(k), int(pos), q.size, k.size, int(head_size), float(rope_base))
        return q, k

    def rope_cos_sin(self, pos, j, head_size, rope_base):
        c, s = C.c_float(), C.c_float()
        self.lib.oracle_rope_cos_sin(int(pos), int(j), int(head_size), float(rope_base), C.byref(c), C.byref(s))
        return c.value, s.value

    def softmax(self, x):
        x = _f32(x).copy()
        self.lib.oracle_softmax(_ptr(x), x.size)
        return x

    def swiglu(self, h1, h3):
        h1, h3 = _f32(h1), _f32(h3)
        out = np.empty_like(h1)
        self.lib.oracle_swiglu(_ptr(out), _ptr(h1), _ptr(h3), h1.size)
        return out

    def kv_index(self, layer, h, pos, off, n_kv_heads, head_size, seq_len) -> int:
        return int(self.lib.oracle_kv_index(layer, h, pos, off, n_kv_heads, head_size, seq_len))

    def sample(self, logits, temperature, penalty, history: Sequence[int], r: float) -> int:
        """Reference sampling semantics on a COPY of logits; returns the token id."""
        buf = _f32(logits).copy()
        hist = np.ascontiguousarray(history, dtype=np.int32)
        hp = hist.ctypes.data_as(_ip) if hist.size else None
        return int(self.lib.oracle_sample(_ptr(buf), buf.size, float(temperature), float(penalty), hp, hist.size,
                                          float(r)))

    def sample_twin(self, logits, temperature, penalty, history: Sequence[int], r: float) -> int:
        """sample() with the CUDA sampler's exp (exp_repro) in place of libm's expf, nothing else changed: what the
        exact-order GPU sampler must reproduce bit for bit."""
        buf = _f32(logits).copy()
        hist = np.ascontiguousarray(history, dtype=np.int32)
        hp = hist.ctypes.data_as(_ip) if hist.size else None
        return int(self.lib.oracle_sample_exp_repro(_ptr(buf), buf.size, float(temperature), float(penalty), hp,
                                                    hist.size, float(r)))

    def rand_floats(self, seed: int, n: int) -> np.ndarray:
        """n values of (float)rand()/(float)RAND_MAX after srand(seed): the reference's r stream."""
        out = np.empty(n, dtype=np.float32)
        self.lib.oracle_srand(int(seed))
        self.lib.oracle_rand_floats(_ptr(out), n)
        return out


class Reference:
    """The compiled, unmodified reference CPU path."""

    def __init__(self):
        if not have_reference():
            raise FileNotFoundError(f"{REF_SO} not built (run `make -C oracle ref` where the reference is)")
        self.lib = lib = C.CDLL(REF_SO)
        lib.ref_load.restype = C.c_void_p
        lib.ref_load.argtypes = [C.c_char_p, C.c_int]
        lib.ref_get_config.argtypes = [C.c_void_p, _ip, _fp]
        lib.ref_forward.restype = C.c_int
        lib.ref_forward.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, _ip, C.c_int]
        lib.ref_srand.argtypes = [C.c_uint]
        lib.ref_rand_floats.argtypes = [_fp, C.c_int]
        lib.ref_sample.restype = C.c_int
        lib.ref_sample.argtypes = [_fp, C.c_int, C.c_float, C.c_float, C.c_float, _ip, C.c_int]
        lib.ref_naive_matmul.argtypes = [_fp, _fp, _fp, C.c_int, C.c_int]
        lib.ref_rmsnorm.argtypes = [_fp, _fp, _fp, C.c_int]
        lib.ref_rope.argtypes = [_fp, _fp, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float]
        lib.ref_softmax.argtypes = [_fp, C.c_int]
        lib.ref_swiglu.argtypes = [_fp, _fp, _fp, C.c_int]
        lib.ref_time_steps.restype = C.c_double
        lib.ref_time_steps.argtypes = [C.c_void_p, _ip, C.c_int, C.c_int, C.c_float, C.c_float, _ip, C.c_int]

    def model(self, cfg, weights) -> "_RefModel":
        return _RefModel(self.lib, cfg, weights)

    def load(self, path: str, seq_len_override: int = 0) -> "_RefModel":
        from lighterpp_b200.formats import ModelConfig
        h = self.lib.ref_load(path.encode(), int(seq_len_override))
        if not h:
            raise RuntimeError(f"reference loader rejected {path}")
        ints = (C.c_int * 8)()
        rb = C.c_float()
        self.lib.ref_get_config(h, ints, C.byref(rb))
        cfg = ModelConfig(*[int(v) for v in ints[:7]], float(rb.value))
        m = _RefModel.__new__(_RefModel)
        m.lib, m.p, m.cfg, m.h, m._w = self.lib, "ref_", cfg, h, {}
        m.weight_precision = int(ints[7])
        m._bind()
        return m

    def matmul(self, x, w):
        x, w = _f32(x), _f32(w)
        out = np.empty(w.shape[0], dtype=np.float32)
        self.lib.ref_naive_matmul(_ptr(out), _ptr(x), _ptr(w), w.shape[0], w.shape[1])
        return out

    def rmsnorm(self, x, weight):
        x, weight = _f32(x), _f32(weight)
        out = np.empty_like(x)
        self.lib.ref_rmsnorm(_ptr(out), _ptr(x), _ptr(weight), x.size)
        return out

    def rope(self, q, k, pos, head_size, rope_base):
        q, k = _f32(q).copy(), _f32(k).copy()
        self.lib.ref_rope(_ptr(q), _ptr(k), int(pos), q.size, k.size, int(head_size), float(rope_base))
        return q, k

    def softmax(self, x):
        x = _f32(x).copy()
        self.lib.ref_softmax(_ptr(x), x.size)
        return x

    def swiglu(self, h1, h3):
        h1, h3 = _f32(h1), _f32(h3)
        out = np.empty_like(h1)
        self.lib.ref_swiglu(_ptr(out), _ptr(h1), _ptr(h3), h1.size)
        return out

    def sample(self, logits, temperature, penalty, history, seed: Optional[int] = None, topp: float = 1.0) -> int:
        """The reference sample() on a COPY; r is the next value of the libc rand() stream."""
        if seed is not None:
            self.lib.ref_srand(int(seed))
        buf = _f32(logits).copy()
        hist = np.ascontiguousarray(history, dtype=np.int32)
        hp = hist.ctypes.data_as(_ip) if hist.size else None
        return int(self.lib.ref_sample(_ptr(buf), buf.size, float(temperature), float(topp), float(penalty), hp,
                                       hist.size))

    def srand(self, seed: int):
        self.lib.ref_srand(int(seed))

    def rand_floats(self, seed: int, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.float32)
        self.lib.ref_srand(int(seed))
        self.lib.ref_rand_floats(_ptr(out), n)
        return out


class _RefModel(_ModelBase):
    def __init__(self, lib, cfg, weights):
        super().__init__(lib, "ref_", cfg, weights)

    def forward(self, token, pos, temperature, penalty, history, topp: float = 1.0) -> int:
        hist = np.ascontiguousarray(history, dtype=np.int32)
        hp = hist.ctypes.data_as(_ip) if hist.size else None
        return int(self.lib.ref_forward(self.h, int(token), int(pos), float(temperature), float(topp),
                                        float(penalty), hp, hist.size))

    def time_steps(self, tokens, start_pos, temperature=0.0, penalty=1.0, history=()) -> float:
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        hist = np.ascontiguousarray(history, dtype=np.int32)
        hp = hist.ctypes.data_as(_ip) if hist.size else None
        return float(self.lib.ref_time_steps(self.h, toks.ctypes.data_as(_ip), toks.size, int(start_pos),
                                             float(temperature), float(penalty), hp, hist.size))
