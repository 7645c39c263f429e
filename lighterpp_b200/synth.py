"""Seeded synthetic models of the benchmark shapes (random-init weights, no real checkpoints).

Every tensor is drawn independently from ``numpy.random.default_rng([seed, tensor_id, layer])`` so a
single layer (or a tensor-parallel rank's share of it) can be generated without materialising the
whole model, and the same bytes come out whichever side (engine, CPU checker, file writer) asks.
Matrices and the embedding are N(0, 0.02) rounded to the model's weight dtype; RMSNorm weights are
1.0, as in the benchmark configurations.
"""
from __future__ import annotations

from typing import Dict, Iterator, Tuple

import numpy as np

from .formats import ModelConfig, tensor_shapes

# name -> (ModelConfig, weight dtype, tied classifier, seed)
SHAPES: Dict[str, Tuple[ModelConfig, str, bool, int]] = {
    # llama2.c stories15M shape; runs on the reference CPU path at full length
    "stories15m": (ModelConfig(288, 768, 6, 6, 6, 32000, 256, 10000.0), "f32", True, 0),
    "tinyllama-1.1b": (ModelConfig(2048, 5632, 22, 32, 4, 32000, 2048, 10000.0), "f16", False, 1),
    "llama-3.2-1b": (ModelConfig(2048, 8192, 16, 32, 8, 128256, 2048, 500000.0), "f16", True, 2),
    "llama-3-8b": (ModelConfig(4096, 14336, 32, 32, 8, 128256, 2048, 500000.0), "f16", False, 3),
    "llama-3-8b-32k": (ModelConfig(4096, 14336, 32, 32, 8, 128256, 33024, 500000.0), "f16", False, 4),
    # small shapes for unit tests (odd head size 48 / GQA factors 1, 2, 4)
    "tiny-f32": (ModelConfig(96, 256, 2, 2, 2, 320, 40, 10000.0), "f32", True, 11),
    "tiny-gqa-f16": (ModelConfig(256, 704, 3, 8, 2, 1000, 96, 500000.0), "f16", False, 12),
    "tiny-tp8-f16": (ModelConfig(512, 1024, 2, 16, 8, 2048, 64, 500000.0), "f16", True, 13),
    # the 8B shape's attention geometry (head size 128, 4 query heads per KV head) at toy width
    "mini-8b-f16": (ModelConfig(1024, 3584, 2, 8, 2, 4096, 128, 500000.0), "f16", False, 14),
    # long-context attention: seq_len large enough to exercise every KV split
    # full-size vocabularies on a toy body: sampler tests
    "vocab32k-f16": (ModelConfig(64, 128, 1, 2, 2, 32000, 16, 10000.0), "f16", True, 16),
    "vocab128k-f16": (ModelConfig(64, 128, 1, 2, 2, 128256, 16, 500000.0), "f16", True, 17),
    "vocab256k-f16": (ModelConfig(64, 128, 1, 2, 2, 256008, 16, 10000.0), "f16", True, 18),
    "vocab50k-f16": (ModelConfig(64, 128, 1, 2, 2, 50264, 16, 10000.0), "f16", True, 19),
    "mini-long-f16": (ModelConfig(512, 1024, 2, 8, 2, 512, 4608, 500000.0), "f16", True, 15),
}

_TENSOR_ID = {"tok_emb": 0, "rms_att": 1, "wq": 2, "wk": 3, "wv": 4, "wo": 5, "rms_ffn": 6, "w1": 7, "w2": 8,
              "w3": 9, "rms_final": 10, "w_cls": 11}
_NORMS = ("rms_att", "rms_ffn", "rms_final")


def np_dtype(name: str):
    return {"f32": np.float32, "f16": np.float16}[name]


def gen_tensor(c: ModelConfig, name: str, seed: int, dtype: str, layer: int = -1, std: float = 0.02) -> np.ndarray:
    """One tensor (``layer=-1`` for unstacked ones, else one layer's slice of a stacked tensor)."""
    shapes = tensor_shapes(c, tied=False)
    shape = shapes[name] if layer < 0 else shapes[name][1:]
    if name in _NORMS:
        return np.ones(shape, dtype=np.float32)
    rng = np.random.default_rng([seed, _TENSOR_ID[name], max(layer, 0)])
    a = rng.standard_normal(shape, dtype=np.float32)
    a *= np.float32(std)
    return a.astype(np_dtype(dtype), copy=False)


def iter_tensors(c: ModelConfig, seed: int, dtype: str, tied: bool) -> Iterator[Tuple[str, int, np.ndarray]]:
    """Yield (name, layer, array) for the whole model, one layer of one tensor at a time."""
    for name, shape in tensor_shapes(c, tied).items():
        if len(shape) == 3 or (len(shape) == 2 and name in ("rms_att", "rms_ffn")):
            for l in range(c.n_layers):
                yield name, l, gen_tensor(c, name, seed, dtype, l)
        else:
            yield name, -1, gen_tensor(c, name, seed, dtype)


def gen_model(c: ModelConfig, seed: int, dtype: str, tied: bool, threads: int = 0) -> Dict[str, np.ndarray]:
    """The whole model as stacked arrays (matrices in ``dtype``, norms FP32).  ``threads`` > 1 draws the
    tensors of different layers on a thread pool (every tensor has its own generator, so the bytes do not
    depend on the number of threads); the billion-parameter shapes need it to be generated in seconds."""
    shapes = tensor_shapes(c, tied)
    out: Dict[str, np.ndarray] = {}
    jobs = []
    for name, shape in shapes.items():
        stacked = len(shape) == 3 or (len(shape) == 2 and name in ("rms_att", "rms_ffn"))
        dt = np.float32 if name in _NORMS else np_dtype(dtype)
        out[name] = np.empty(shape, dtype=dt)
        for l in (range(c.n_layers) if stacked else [-1]):
            jobs.append((name, l))

    def fill(job):
        name, l = job
        if l < 0:
            out[name][...] = gen_tensor(c, name, seed, dtype)
        else:
            out[name][l] = gen_tensor(c, name, seed, dtype, l)

    if threads > 1:
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(threads) as pool:
            list(pool.map(fill, jobs))
    else:
        for job in jobs:
            fill(job)
    return out


def named(name: str) -> Tuple[ModelConfig, str, bool, int, Dict[str, np.ndarray]]:
    c, dtype, tied, seed = SHAPES[name]
    return c, dtype, tied, seed, gen_model(c, seed, dtype, tied)


def as_f32(tensors: Dict[str, np.ndarray]) -> Dict[str, np.ndarray]:
    """Exact widening of every tensor to FP32 (what the reference's GGUF loader does on the host,
    src/loader.cpp:346-402): the arrays the CPU checkers consume."""
    return {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in tensors.items()}


def prompt_tokens(vocab_size: int, n: int, seed: int) -> np.ndarray:
    return np.random.default_rng([seed, 1000]).integers(0, vocab_size, size=n, dtype=np.int32)
