"""Tensor-parallel partition of the decode step (host-side description of what each rank holds).

Rank r of N owns query heads [r*H/N, (r+1)*H/N), KV heads [r*KVH/N, ...) -- GQA groups stay intact
because kv_head = h / (H/KVH) (src/model.cpp:180) -- and FFN columns [r*F/N, ...).  Row slices
(wq/wk/wv/w1/w3) produce this rank's part of an activation; column slices (wo/w2) consume it and
produce a partial sum of the full output, which one all-reduce(sum) over the ranks completes.  The
embedding, norms, classifier and sampler are replicated.  The engine applies the same slicing on
the device in lpp_upload_tensor; this module is the reference description used by hosts that
pre-shard and by the CPU tests of the multi-rank path.
"""
from __future__ import annotations

from typing import Dict

import numpy as np

from .formats import ModelConfig

ROW_SLICED = ("wq", "wk", "wv", "w1", "w3")
COL_SLICED = ("wo", "w2")


def validate(c: ModelConfig, tp_size: int) -> None:
    if tp_size < 1:
        raise ValueError("tp_size must be >= 1")
    if c.n_kv_heads % tp_size or c.hidden_dim % tp_size:
        raise ValueError(f"tp_size {tp_size} must divide n_kv_heads {c.n_kv_heads} and hidden_dim {c.hidden_dim}")


def shard_layer_tensor(c: ModelConfig, name: str, a: np.ndarray, rank: int, tp_size: int) -> np.ndarray:
    """This rank's share of one layer's tensor ``a`` (reference layout [rows][cols])."""
    validate(c, tp_size)
    if not 0 <= rank < tp_size:
        raise ValueError("rank out of range")
    if name in ROW_SLICED:
        n = a.shape[0] // tp_size
        return a[rank * n:(rank + 1) * n]
    if name in COL_SLICED:
        n = a.shape[1] // tp_size
        return a[:, rank * n:(rank + 1) * n]
    return a  # replicated


def shard_model(c: ModelConfig, tensors: Dict[str, np.ndarray], rank: int, tp_size: int) -> Dict[str, np.ndarray]:
    out = {}
    for name, a in tensors.items():
        if name in ROW_SLICED or name in COL_SLICED:
            out[name] = np.stack([shard_layer_tensor(c, name, a[l], rank, tp_size) for l in range(c.n_layers)])
        else:
            out[name] = a
    return out


def local_config(c: ModelConfig, tp_size: int) -> Dict[str, int]:
    validate(c, tp_size)
    return {"n_heads": c.n_heads // tp_size, "n_kv_heads": c.n_kv_heads // tp_size,
            "q_rows": c.dim // tp_size, "kv_rows": c.kv_dim // tp_size, "ffn_cols": c.hidden_dim // tp_size}
