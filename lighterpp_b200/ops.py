"""The reference's per-operator host wrappers (src/kernels.cuh:24-36) over the C ABI, for torch CUDA tensors.

Same names and argument meaning as the reference; tensors stand in for raw device pointers.  Work is
queued on torch's current stream; nothing here synchronises.  There is no CPU path.
"""
from __future__ import annotations

import ctypes as C

import torch

from .engine import LPP_F16, LPP_F32, _check, load_library

WEIGHT_FP32, WEIGHT_FP16 = 0, 1  # src/model.h:8-12


def _p(t: torch.Tensor) -> C.c_void_p:
    if not t.is_cuda or not t.is_contiguous():
        raise ValueError("expected a contiguous CUDA tensor")
    return C.c_void_p(t.data_ptr())


def _s() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _lib():
    lib = load_library()
    if not getattr(lib, "_ops_bound", False):
        vp, i, f, i64 = C.c_void_p, C.c_int, C.c_float, C.c_int64
        lib.lpp_op_convert_f32_to_f16.argtypes = [vp, vp, i64, vp]
        lib.lpp_op_gemv.argtypes = [vp, vp, vp, i, i, i, vp]
        lib.lpp_op_rmsnorm.argtypes = [vp, vp, vp, i, vp]
        lib.lpp_op_rope.argtypes = [vp, vp, i, i, i, i, f, vp]
        lib.lpp_op_swiglu.argtypes = [vp, vp, vp, i, vp]
        lib.lpp_op_softmax_multihead.argtypes = [vp, vp, i, i, i, vp]
        lib.lpp_op_scale_multihead.argtypes = [vp, f, i, i, i, vp]
        lib.lpp_op_aggregation_multihead.argtypes = [vp, vp, vp, i, i, i, i, i, vp]
        lib.lpp_op_residual_add.argtypes = [vp, vp, vp, i, vp]
        lib.lpp_op_scatter_kv.argtypes = [vp, vp, vp, vp, i, i, i, i, i, vp]
        lib.lpp_op_multihead_gemv.argtypes = [vp, vp, vp, i, i, i, i, i, i, vp]
        lib.lpp_op_rope_scatter.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, f, vp]
        lib.lpp_op_sample.argtypes = [vp, i, f, f, vp, i, f, vp, vp]
        lib._ops_bound = True
    return lib


def cuda_convert_f32_to_f16(dst, src, n):
    _check(_lib().lpp_op_convert_f32_to_f16(_p(dst), _p(src), int(n), _s()), "cuda_convert_f32_to_f16")


def cuda_gemv(d_out, d_x, d_w, n, d, precision):
    """out[n] = w[n,d] . x[d]; ``precision`` is WEIGHT_FP32 / WEIGHT_FP16.  No workspace argument: x is never
    rounded to FP16 (the reference needs one for that, src/matmul.cu:136-141)."""
    _check(_lib().lpp_op_gemv(_p(d_out), _p(d_x), _p(d_w), int(n), int(d), LPP_F16 if precision == WEIGHT_FP16 else LPP_F32,
                              _s()), "cuda_gemv")


def cuda_rmsnorm(d_out, d_x, d_w, n):
    _check(_lib().lpp_op_rmsnorm(_p(d_out), _p(d_x), _p(d_w), int(n), _s()), "cuda_rmsnorm")


def cuda_rope(d_q, d_k, pos, dim, kv_dim, head_size, rope_base):
    _check(_lib().lpp_op_rope(_p(d_q), _p(d_k), int(pos), int(dim), int(kv_dim), int(head_size), float(rope_base), _s()),
           "cuda_rope")


def cuda_swiglu(d_hb, d_h1, d_h3, size):
    _check(_lib().lpp_op_swiglu(_p(d_hb), _p(d_h1), _p(d_h3), int(size), _s()), "cuda_swiglu")


def cuda_softmax_multihead(d_out, d_x, n_heads, seq_len, att_stride):
    _check(_lib().lpp_op_softmax_multihead(_p(d_out), _p(d_x), int(n_heads), int(seq_len), int(att_stride), _s()),
           "cuda_softmax_multihead")


def cuda_scale_multihead(d_att, scale, n_heads, seq_len, att_stride):
    _check(_lib().lpp_op_scale_multihead(_p(d_att), float(scale), int(n_heads), int(seq_len), int(att_stride), _s()),
           "cuda_scale_multihead")


def cuda_aggregation_multihead(d_out, d_v, d_att, n_heads, seq_len, head_size, gqa_factor, att_stride):
    _check(_lib().lpp_op_aggregation_multihead(_p(d_out), _p(d_v), _p(d_att), int(n_heads), int(seq_len), int(head_size),
                                               int(gqa_factor), int(att_stride), _s()), "cuda_aggregation_multihead")


def cuda_residual_add(d_out, d_a, d_b, n):
    _check(_lib().lpp_op_residual_add(_p(d_out), _p(d_a), _p(d_b), int(n), _s()), "cuda_residual_add")


def cuda_scatter_kv(d_key_cache, d_value_cache, d_k, d_v, layer, pos, n_kv_heads, head_size, seq_len):
    _check(_lib().lpp_op_scatter_kv(_p(d_key_cache), _p(d_value_cache), _p(d_k), _p(d_v), int(layer), int(pos),
                                    int(n_kv_heads), int(head_size), int(seq_len), _s()), "cuda_scatter_kv")


def cuda_multihead_gemv(d_out, d_q, d_k_cache, layer, pos, n_heads, n_kv_heads, head_size, seq_len):
    _check(_lib().lpp_op_multihead_gemv(_p(d_out), _p(d_q), _p(d_k_cache), int(layer), int(pos), int(n_heads),
                                        int(n_kv_heads), int(head_size), int(seq_len), _s()), "cuda_multihead_gemv")


def cuda_rope_scatter(d_q, d_k, d_v, d_key_cache, d_value_cache, layer, pos, dim, n_kv_heads, head_size, seq_len,
                      rope_base):
    _check(_lib().lpp_op_rope_scatter(_p(d_q), _p(d_k), _p(d_v), _p(d_key_cache), _p(d_value_cache), int(layer),
                                      int(pos), int(dim), int(n_kv_heads), int(head_size), int(seq_len),
                                      float(rope_base), _s()), "cuda_rope_scatter")


def cuda_sample(d_logits, vocab_size, temperature, penalty, d_history, history_len, r, d_sampled_token):
    """``r`` is passed in (the reference wrapper draws it from rand(), src/sample.cu:211)."""
    hp = _p(d_history) if d_history is not None and history_len > 0 else C.c_void_p(None)
    _check(_lib().lpp_op_sample(_p(d_logits), int(vocab_size), float(temperature), float(penalty), hp, int(history_len),
                                float(r), _p(d_sampled_token), _s()), "cuda_sample")
