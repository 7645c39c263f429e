"""Python host over the C ABI of ``liblpp_b200.so`` (``include/lpp_b200.h``).

``Engine`` mirrors the reference's model-step interface -- ``malloc_run_state`` / ``forward(token, pos,
..., temperature, topp, penalty, history, history_len)`` / ``free_run_state`` (src/model.h:117-164) --
with the same argument meaning.  There is no CPU fallback: if the CUDA library is missing or no
sm_100 device is present, construction raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, Iterable, Optional, Sequence, Tuple

import numpy as np

from .formats import ModelConfig

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liblpp_b200.so")

LPP_F32, LPP_F16 = 0, 1
MEM_HOST, MEM_DEVICE = 0, 1
FLAG_GEMV_LDG, FLAG_NO_PDL, FLAG_NO_GRAPH, FLAG_FAST_SAMPLER = 1, 2, 4, 16
TENSOR_IDS = {"tok_emb": 0, "rms_att": 1, "wq": 2, "wk": 3, "wv": 4, "wo": 5, "rms_ffn": 6, "w1": 7, "w2": 8,
              "w3": 9, "rms_final": 10, "w_cls": 11}
_UNSTACKED = ("tok_emb", "rms_final", "w_cls")
TP_HANDLE_BYTES = 64
FLAG_TP_NCCL, FLAG_TP_LOCAL, FLAG_NO_PREFILL_GEMM = 32, 64, 128
KINDS = ["qkv_gemv", "attention", "oproj_gemv", "gateup_gemv", "down_gemv", "lmhead_gemv", "sampler", "allreduce",
         "reserved8", "reserved9"]

# every symbol include/lpp_b200.h declares; tests check the built library exports all of them
EXPORTS = [
    "lpp_engine_create", "lpp_engine_destroy", "lpp_nccl_unique_id", "lpp_upload_tensor", "lpp_finalize",
    "lpp_step", "lpp_step_logits", "lpp_decode", "lpp_prefill", "lpp_sample_logits", "lpp_kv_prefill", "lpp_kv_read",
    "lpp_kv_index", "lpp_strerror", "lpp_last_error", "lpp_engine_stream", "lpp_kernels_per_step",
    "lpp_step_bytes", "lpp_profile_step", "lpp_profile_kind", "lpp_tp_export", "lpp_tp_connect", "lpp_op_convert_f32_to_f16", "lpp_op_gemv", "lpp_op_rmsnorm",
    "lpp_op_rope", "lpp_op_swiglu", "lpp_op_softmax_multihead", "lpp_op_scale_multihead",
    "lpp_op_aggregation_multihead", "lpp_op_residual_add", "lpp_op_scatter_kv", "lpp_op_multihead_gemv",
    "lpp_op_rope_scatter", "lpp_op_sample", "lpp_op_sample_static",
]


class LppError(RuntimeError):
    def __init__(self, status: int, what: str, detail: str):
        super().__init__(f"{what}: status {status} ({detail})")
        self.status = status


class Config(C.Structure):
    _fields_ = [("dim", C.c_int32), ("hidden_dim", C.c_int32), ("n_layers", C.c_int32), ("n_heads", C.c_int32),
                ("n_kv_heads", C.c_int32), ("vocab_size", C.c_int32), ("seq_len", C.c_int32),
                ("rope_base", C.c_float), ("weight_dtype", C.c_int32), ("kv_dtype", C.c_int32),
                ("tp_rank", C.c_int32), ("tp_size", C.c_int32), ("device", C.c_int32), ("flags", C.c_uint32),
                ("ring_kb", C.c_int32), ("attn_splits", C.c_int32), ("wait_ms", C.c_int32), ("tp_wait_ms", C.c_int32)]


class SampleParams(C.Structure):
    _fields_ = [("temperature", C.c_float), ("penalty", C.c_float)]


_lib = None


def load_library() -> C.CDLL:
    """Load the CUDA library; raise (never fall back) when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise FileNotFoundError(
            f"{LIB_PATH} is missing: build it with lighterpp_b200/csrc/build.sh (or __graft_entry__.build()); "
            "this package has no CPU fallback")
    lib = C.CDLL(LIB_PATH)
    vp, ip, fp = C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_float)
    lib.lpp_engine_create.argtypes = [C.POINTER(Config), vp, C.POINTER(vp)]
    lib.lpp_engine_destroy.argtypes = [vp]
    lib.lpp_nccl_unique_id.argtypes = [vp]
    lib.lpp_upload_tensor.argtypes = [vp, C.c_int, C.c_int, vp, C.c_int, C.c_int]
    lib.lpp_finalize.argtypes = [vp]
    lib.lpp_step.argtypes = [vp, C.c_int, C.c_int, C.POINTER(SampleParams), ip, C.c_int, C.c_float, ip]
    lib.lpp_step_logits.argtypes = [vp, C.c_int, C.c_int, fp]
    lib.lpp_decode.argtypes = [vp, C.c_int, C.c_int, C.c_int, C.POINTER(SampleParams), ip, C.c_int, C.c_int, fp, ip,
                               fp]
    lib.lpp_sample_logits.argtypes = [vp, fp, C.POINTER(SampleParams), ip, C.c_int, C.c_float, ip]
    lib.lpp_prefill.argtypes = [vp, ip, C.c_int, C.c_int, fp]
    lib.lpp_kv_prefill.argtypes = [vp, C.c_int, vp, vp, C.c_int, C.c_int, C.c_int]
    lib.lpp_kv_read.argtypes = [vp, C.c_int, C.c_int, C.c_int, fp, fp]
    lib.lpp_kv_index.argtypes = [vp, C.c_int, C.c_int, C.c_int, C.c_int]
    lib.lpp_kv_index.restype = C.c_int64
    lib.lpp_strerror.argtypes = [C.c_int]
    lib.lpp_strerror.restype = C.c_char_p
    lib.lpp_last_error.restype = C.c_char_p
    lib.lpp_engine_stream.argtypes = [vp]
    lib.lpp_engine_stream.restype = vp
    lib.lpp_kernels_per_step.argtypes = [vp]
    lib.lpp_step_bytes.argtypes = [vp, C.c_int]
    lib.lpp_step_bytes.restype = C.c_int64
    lib.lpp_profile_step.argtypes = [vp, C.c_int, C.c_int, C.POINTER(SampleParams), fp, ip, C.POINTER(C.c_int64)]
    lib.lpp_profile_kind.argtypes = [vp, C.c_int, C.c_int, C.c_int, fp, ip]
    lib.lpp_tp_export.argtypes = [vp, vp, C.c_size_t]
    lib.lpp_tp_connect.argtypes = [vp, vp, C.c_size_t]
    _lib = lib
    return lib


def _check(status: int, what: str) -> None:
    if status != 0:
        lib = load_library()
        raise LppError(status, what, f"{lib.lpp_strerror(status).decode()}: {lib.lpp_last_error().decode()}")


def nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    _check(load_library().lpp_nccl_unique_id(buf), "lpp_nccl_unique_id")
    return buf.raw


def _np_dtype_code(a: np.ndarray) -> int:
    if a.dtype == np.float32:
        return LPP_F32
    if a.dtype == np.float16:
        return LPP_F16
    raise TypeError(f"unsupported dtype {a.dtype}")


class Engine:
    """One tensor-parallel rank of the decode engine on one GPU."""

    def __init__(self, cfg: ModelConfig, weight_dtype: str = "f16", kv_dtype: str = "f16", *, device: int = 0,
                 tp_rank: int = 0, tp_size: int = 1, nccl_id: Optional[bytes] = None, flags: int = 0,
                 ring_kb: int = 0, attn_splits: int = 0, wait_ms: int = 0, tp_wait_ms: int = 0):
        self.lib = load_library()
        self.cfg = cfg
        self.weight_dtype = {"f32": LPP_F32, "f16": LPP_F16}[weight_dtype]
        c = Config(cfg.dim, cfg.hidden_dim, cfg.n_layers, cfg.n_heads, cfg.n_kv_heads, cfg.vocab_size, cfg.seq_len,
                   cfg.rope_base, self.weight_dtype, {"f32": LPP_F32, "f16": LPP_F16}[kv_dtype], tp_rank, tp_size,
                   device, flags, ring_kb, attn_splits, wait_ms, tp_wait_ms)
        self.tp_rank, self.tp_size = tp_rank, tp_size
        h = C.c_void_p()
        idbuf = C.create_string_buffer(nccl_id, 128) if nccl_id is not None else None
        _check(self.lib.lpp_engine_create(C.byref(c), idbuf, C.byref(h)), "lpp_engine_create")
        self.h = h

    # ---- weights -------------------------------------------------------------------------------
    def upload(self, name: str, array, layer: int = 0) -> None:
        """``array``: a numpy array (host) or a torch CUDA tensor (device), the FULL reference-layout tensor of
        one layer (or an unstacked tensor); the engine keeps this rank's share."""
        tid = TENSOR_IDS[name]
        if isinstance(array, np.ndarray):
            a = np.ascontiguousarray(array)
            ptr, code, kind = a.ctypes.data, _np_dtype_code(a), MEM_HOST
        else:  # torch tensor on the engine's device
            import torch
            a = array.contiguous()
            code = {torch.float32: LPP_F32, torch.float16: LPP_F16}[a.dtype]
            ptr, kind = a.data_ptr(), (MEM_DEVICE if a.is_cuda else MEM_HOST)
            if a.is_cuda:
                torch.cuda.current_stream(a.device).synchronize()
        _check(self.lib.lpp_upload_tensor(self.h, tid, layer, C.c_void_p(ptr), code, kind), f"upload {name}[{layer}]")

    def load_weights(self, tensors: Dict[str, np.ndarray]) -> None:
        """Upload stacked reference-layout tensors (see ``formats.tensor_shapes``) and finalize."""
        for name, a in tensors.items():
            if name in _UNSTACKED or a.ndim == 1:
                self.upload(name, a)
            else:
                for l in range(a.shape[0]):
                    self.upload(name, a[l], l)
        self.finalize()

    def finalize(self) -> None:
        _check(self.lib.lpp_finalize(self.h), "lpp_finalize")

    # ---- the hot path --------------------------------------------------------------------------
    def forward(self, token: int, pos: int, temperature: float = 0.0, penalty: float = 1.0,
                history: Sequence[int] = (), r: float = 0.0) -> int:
        """``forward(token, pos, ...)`` of src/model.cpp:342-384; ``r`` replaces the ``rand()`` draw."""
        sp = SampleParams(temperature, penalty)
        hist = np.ascontiguousarray(history, dtype=np.int32)
        out = C.c_int(-1)
        hp = hist.ctypes.data_as(C.POINTER(C.c_int)) if hist.size else None
        _check(self.lib.lpp_step(self.h, int(token), int(pos), C.byref(sp), hp, int(hist.size), float(r),
                                 C.byref(out)), "lpp_step")
        return out.value

    def step_logits(self, token: int, pos: int) -> np.ndarray:
        out = np.empty(self.cfg.vocab_size, dtype=np.float32)
        _check(self.lib.lpp_step_logits(self.h, int(token), int(pos), out.ctypes.data_as(C.POINTER(C.c_float))),
               "lpp_step_logits")
        return out

    def decode(self, first_token: int, start_pos: int, n: int, temperature: float = 0.0, penalty: float = 1.0,
               history: Sequence[int] = (), history_window: int = 64, r: Optional[np.ndarray] = None
               ) -> Tuple[np.ndarray, float]:
        """The generate loop of src/main.cpp:199-223 on the device; returns (tokens[n], device milliseconds)."""
        sp = SampleParams(temperature, penalty)
        hist = np.ascontiguousarray(history, dtype=np.int32)
        hp = hist.ctypes.data_as(C.POINTER(C.c_int)) if hist.size else None
        rv = None if r is None else np.ascontiguousarray(r, dtype=np.float32)
        if rv is not None and rv.size < n:
            raise ValueError("need one r per step")
        out = np.empty(n, dtype=np.int32)
        ms = C.c_float(0)
        _check(self.lib.lpp_decode(self.h, int(first_token), int(start_pos), int(n), C.byref(sp), hp, int(hist.size),
                                   int(history_window),
                                   rv.ctypes.data_as(C.POINTER(C.c_float)) if rv is not None else None,
                                   out.ctypes.data_as(C.POINTER(C.c_int)), C.byref(ms)), "lpp_decode")
        return out, ms.value

    def prefill(self, tokens: Sequence[int], start_pos: int = 0) -> float:
        """The prompt loop of src/main.cpp:163-179 as one batched pass: fills the K/V cache for ``tokens`` at positions
        ``start_pos ..`` (no logits; the last prompt token still goes through ``forward``).  Returns device ms."""
        toks = np.ascontiguousarray(tokens, dtype=np.int32)
        ms = C.c_float(0)
        _check(self.lib.lpp_prefill(self.h, toks.ctypes.data_as(C.POINTER(C.c_int)), int(toks.size), int(start_pos),
                                    C.byref(ms)), "lpp_prefill")
        return ms.value

    def sample(self, logits: np.ndarray, temperature: float, penalty: float = 1.0, history: Sequence[int] = (),
               r: float = 0.0) -> int:
        """``cuda_sample`` (src/sample.cu:210-214) on given logits."""
        lg = np.ascontiguousarray(logits, dtype=np.float32)
        if lg.size != self.cfg.vocab_size:
            raise ValueError("logits size != vocab_size")
        sp = SampleParams(temperature, penalty)
        hist = np.ascontiguousarray(history, dtype=np.int32)
        hp = hist.ctypes.data_as(C.POINTER(C.c_int)) if hist.size else None
        out = C.c_int(-1)
        _check(self.lib.lpp_sample_logits(self.h, lg.ctypes.data_as(C.POINTER(C.c_float)), C.byref(sp), hp,
                                          int(hist.size), float(r), C.byref(out)), "lpp_sample_logits")
        return out.value

    # ---- KV cache ------------------------------------------------------------------------------
    def kv_prefill(self, layer: int, k, v, n_pos: int) -> None:
        """k, v: [n_kv_heads][n_pos][head_size] numpy arrays or torch CUDA tensors (f16/f32)."""
        if isinstance(k, np.ndarray):
            k, v = np.ascontiguousarray(k), np.ascontiguousarray(v)
            kp, vp_, code, kind = k.ctypes.data, v.ctypes.data, _np_dtype_code(k), MEM_HOST
        else:
            import torch
            k, v = k.contiguous(), v.contiguous()
            code = {torch.float32: LPP_F32, torch.float16: LPP_F16}[k.dtype]
            kp, vp_, kind = k.data_ptr(), v.data_ptr(), MEM_DEVICE
            torch.cuda.current_stream(k.device).synchronize()
        _check(self.lib.lpp_kv_prefill(self.h, layer, C.c_void_p(kp), C.c_void_p(vp_), int(n_pos), code, kind),
               "lpp_kv_prefill")

    def kv_read(self, layer: int, kv_head: int, pos: int) -> Tuple[np.ndarray, np.ndarray]:
        hs = self.cfg.head_size
        k, v = np.empty(hs, dtype=np.float32), np.empty(hs, dtype=np.float32)
        fp = C.POINTER(C.c_float)
        _check(self.lib.lpp_kv_read(self.h, layer, kv_head, pos, k.ctypes.data_as(fp), v.ctypes.data_as(fp)),
               "lpp_kv_read")
        return k, v

    def kv_index(self, layer: int, kv_head: int, pos: int, off: int) -> int:
        return int(self.lib.lpp_kv_index(self.h, layer, kv_head, pos, off))

    # ---- introspection -------------------------------------------------------------------------
    @property
    def stream(self) -> int:
        return int(self.lib.lpp_engine_stream(self.h) or 0)

    @property
    def kernels_per_step(self) -> int:
        return int(self.lib.lpp_kernels_per_step(self.h))

    def step_bytes(self, pos: int) -> int:
        return int(self.lib.lpp_step_bytes(self.h, int(pos)))

    def profile_step(self, pos: int, iters: int = 5, temperature: float = 0.0, penalty: float = 1.0
                     ) -> Dict[str, Dict[str, float]]:
        """Isolated per-kernel-kind durations of one step; the sampler runs with the given parameters."""
        ms = (C.c_float * 10)()
        n = (C.c_int * 10)()
        b = (C.c_int64 * 10)()
        sp = SampleParams(temperature, penalty)
        _check(self.lib.lpp_profile_step(self.h, int(pos), int(iters), C.byref(sp), ms, n, b), "lpp_profile_step")
        return {KINDS[i]: {"ms": float(ms[i]), "launches": int(n[i]), "bytes": int(b[i])} for i in range(10)}

    def tp_export(self) -> bytes:
        """IPC handle of this rank's exchange buffer (to be gathered over the caller's host channel)."""
        buf = C.create_string_buffer(TP_HANDLE_BYTES)
        _check(self.lib.lpp_tp_export(self.h, buf, TP_HANDLE_BYTES), "lpp_tp_export")
        return buf.raw

    def tp_connect(self, handles: Sequence[bytes]) -> None:
        """Maps every rank's exchange buffer (handles in rank order); call before the weights are finalized."""
        if len(handles) != self.tp_size or any(len(h) != TP_HANDLE_BYTES for h in handles):
            raise ValueError("need one %d-byte handle per rank, in rank order" % TP_HANDLE_BYTES)
        blob = C.create_string_buffer(b"".join(handles), TP_HANDLE_BYTES * self.tp_size)
        _check(self.lib.lpp_tp_connect(self.h, blob, TP_HANDLE_BYTES), "lpp_tp_connect")

    def profile_kind(self, pos: int, kind: str, iters: int = 5) -> Dict[str, float]:
        """Average launch duration of one kernel kind, its launches of a step run back to back."""
        ms = C.c_float(0.0)
        n = C.c_int(0)
        _check(self.lib.lpp_profile_kind(self.h, int(pos), KINDS.index(kind), int(iters), C.byref(ms), C.byref(n)),
               "lpp_profile_kind")
        return {"ms_per_launch": float(ms.value), "launches": int(n.value)}

    def close(self) -> None:
        if getattr(self, "h", None):
            self.lib.lpp_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def engine_from_file(path: str, **kw) -> Engine:
    """Load a llama2.c ``.bin`` or GGUF model file into a new engine (src/main.cpp:44-113 dispatch)."""
    from .formats import load_model
    cfg, tensors = load_model(path)
    wd = "f16" if tensors["wq"].dtype == np.float16 else "f32"
    kw.setdefault("kv_dtype", "f16" if wd == "f16" else "f32")
    e = Engine(cfg, wd, **kw)
    e.load_weights(tensors)
    return e
