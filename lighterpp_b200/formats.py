"""Model-file formats on either side of the decode path: llama2.c ``.bin`` and GGUF (F32/F16).

These are the two checkpoint formats Lighter++ reads (llama2.c: src/loader.cpp:134-172 with the
tensor order of src/loader.cpp:18-66; GGUF v2/v3: src/gguf.cpp:123-270 and the tensor names of
src/loader.cpp:456-540).  The writers produce files the reference's unmodified loaders accept; the
readers feed the B200 engine through the C ABI.  Everything here is host-side numpy; no CUDA.

Tensor naming used throughout this package (one name per reference ``transformerWeights`` member):

    tok_emb [V,D]  rms_att [L,D]  wq [L,D,D]  wk [L,KV,D]  wv [L,KV,D]  wo [L,D,D]
    rms_ffn [L,D]  w1 [L,F,D]     w2 [L,D,F]  w3 [L,F,D]   rms_final [D]  w_cls [V,D] (optional)
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, asdict
from typing import Dict, Iterable, Optional, Tuple

import numpy as np

GGUF_MAGIC = 0x46554747
GGML_F32, GGML_F16 = 0, 1
(T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64) = range(13)
_SCALAR = {T_U8: "<B", T_I8: "<b", T_U16: "<H", T_I16: "<h", T_U32: "<I", T_I32: "<i", T_F32: "<f",
           T_BOOL: "<?", T_U64: "<Q", T_I64: "<q", T_F64: "<d"}


@dataclass
class ModelConfig:
    """Mirror of the reference ``Config`` (src/model.h:21-31) without the precision enum."""
    dim: int
    hidden_dim: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    vocab_size: int
    seq_len: int
    rope_base: float = 10000.0

    @property
    def head_size(self) -> int:
        return self.dim // self.n_heads

    @property
    def kv_dim(self) -> int:
        return self.dim * self.n_kv_heads // self.n_heads

    def asdict(self):
        return asdict(self)


def tensor_shapes(c: ModelConfig, tied: bool) -> Dict[str, Tuple[int, ...]]:
    L, D, F, V, KV = c.n_layers, c.dim, c.hidden_dim, c.vocab_size, c.kv_dim
    s = {"tok_emb": (V, D), "rms_att": (L, D), "wq": (L, D, D), "wk": (L, KV, D), "wv": (L, KV, D),
         "wo": (L, D, D), "rms_ffn": (L, D), "w1": (L, F, D), "w2": (L, D, F), "w3": (L, F, D),
         "rms_final": (D,)}
    if not tied:
        s["w_cls"] = (V, D)
    return s


# --------------------------------------------------------------------------- llama2.c .bin

_BIN_ORDER = ["tok_emb", "rms_att", "wq", "wk", "wv", "wo", "rms_ffn", "w1", "w2", "w3", "rms_final"]


def write_llama2c_bin(path: str, c: ModelConfig, tensors: Dict[str, np.ndarray]) -> None:
    """28-byte header of 7 int32 then FP32 tensors in the order src/loader.cpp:21-63 carves them.

    The reference always treats ``.bin`` files as tied (src/loader.cpp:66), so ``w_cls`` is not
    written.  Eight zero bytes are appended because the reference copies a 36-byte ``Config`` out
    of the 28-byte header (src/loader.cpp:158-159) and a file that ended exactly at the last
    weight would still be fine, but a tiny test file smaller than 36 bytes would not.
    """
    shapes = tensor_shapes(c, tied=True)
    with open(path, "wb") as f:
        f.write(struct.pack("<7i", c.dim, c.hidden_dim, c.n_layers, c.n_heads, c.n_kv_heads, c.vocab_size,
                            c.seq_len))
        for name in _BIN_ORDER:
            a = np.ascontiguousarray(tensors[name], dtype=np.float32)
            assert a.shape == shapes[name], (name, a.shape, shapes[name])
            a.tofile(f)
        f.write(b"\0" * 8)


def read_llama2c_bin(path: str) -> Tuple[ModelConfig, Dict[str, np.ndarray]]:
    raw = np.memmap(path, dtype=np.uint8, mode="r")
    if raw.size < 28:
        raise ValueError(f"{path}: shorter than the 28-byte llama2.c header")
    hdr = struct.unpack("<7i", bytes(raw[:28]))
    if min(hdr[:5]) <= 0 or hdr[5] == 0 or hdr[6] <= 0 or hdr[0] % hdr[3] or hdr[3] % hdr[4]:
        raise ValueError(f"{path}: implausible llama2.c header {hdr}")
    # llama2.c marks an untied classifier with a negative vocab size; Lighter++ ignores that
    # (src/loader.cpp:66) and so do we, but the magnitude is the real vocabulary size.
    c = ModelConfig(hdr[0], hdr[1], hdr[2], hdr[3], hdr[4], abs(hdr[5]), hdr[6], 10000.0)
    shapes = tensor_shapes(c, tied=True)
    need = 28 + 4 * sum(int(np.prod(shapes[n])) for n in _BIN_ORDER)
    if raw.size < need:
        raise ValueError(f"{path}: truncated ({raw.size} bytes, need {need})")
    out, off = {}, 28
    for name in _BIN_ORDER:
        n = int(np.prod(shapes[name]))
        out[name] = np.frombuffer(raw, dtype=np.float32, count=n, offset=off).reshape(shapes[name])
        off += 4 * n
    return c, out


# --------------------------------------------------------------------------- GGUF

def _gguf_str(s: str) -> bytes:
    b = s.encode("utf-8")
    return struct.pack("<Q", len(b)) + b


def _gguf_kv(key: str, typ: int, value) -> bytes:
    out = _gguf_str(key) + struct.pack("<I", typ)
    if typ == T_STR:
        return out + _gguf_str(value)
    if typ == T_ARR:
        etyp, items = value
        out += struct.pack("<IQ", etyp, len(items))
        if etyp == T_STR:
            return out + b"".join(_gguf_str(s) for s in items)
        return out + b"".join(struct.pack(_SCALAR[etyp], v) for v in items)
    return out + struct.pack(_SCALAR[typ], value)


def _gguf_tensor_names(c: ModelConfig, tied: bool) -> Iterable[Tuple[str, str, Optional[int]]]:
    """(gguf name, our name, layer or None) in file order."""
    yield "token_embd.weight", "tok_emb", None
    if not tied:
        yield "output.weight", "w_cls", None
    yield "output_norm.weight", "rms_final", None
    per_layer = [("attn_norm", "rms_att"), ("attn_q", "wq"), ("attn_k", "wk"), ("attn_v", "wv"),
                 ("attn_output", "wo"), ("ffn_norm", "rms_ffn"), ("ffn_gate", "w1"), ("ffn_down", "w2"),
                 ("ffn_up", "w3")]
    for l in range(c.n_layers):
        for g, ours in per_layer:
            yield f"blk.{l}.{g}.weight", ours, l


def write_gguf(path: str, c: ModelConfig, tensors: Dict[str, np.ndarray], *, version: int = 3,
               arch: str = "llama", alignment: int = 32) -> None:
    """Minimal GGUF the reference parser accepts (src/gguf.cpp:123-270, src/loader.cpp:213-334).

    Hyper-parameters must be UINT32 (src/gguf.cpp:316-319), ``rope.freq_base`` FLOAT32, and the
    vocabulary size is the length of ``tokenizer.ggml.tokens`` (src/loader.cpp:300-307).  Matrices
    keep the dtype of the arrays passed in (float16 -> F16, float32 -> F32); 1-D norm weights are
    always written as F32.  Tied embeddings = no ``w_cls`` entry (src/loader.cpp:464-472).
    """
    tied = "w_cls" not in tensors
    kv = [
        _gguf_kv("general.architecture", T_STR, arch),
        _gguf_kv(f"{arch}.embedding_length", T_U32, c.dim),
        _gguf_kv(f"{arch}.feed_forward_length", T_U32, c.hidden_dim),
        _gguf_kv(f"{arch}.block_count", T_U32, c.n_layers),
        _gguf_kv(f"{arch}.attention.head_count", T_U32, c.n_heads),
        _gguf_kv(f"{arch}.attention.head_count_kv", T_U32, c.n_kv_heads),
        _gguf_kv(f"{arch}.context_length", T_U32, c.seq_len),
        _gguf_kv(f"{arch}.rope.freq_base", T_F32, float(c.rope_base)),
        _gguf_kv("tokenizer.ggml.model", T_STR, "llama"),
        _gguf_kv("tokenizer.ggml.tokens", T_ARR, (T_STR, [f"t{i}" for i in range(c.vocab_size)])),
    ]
    infos, blobs, off = [], [], 0
    for gname, ours, layer in _gguf_tensor_names(c, tied):
        a = tensors[ours] if layer is None else tensors[ours][layer]
        if a.ndim == 1:
            a = np.ascontiguousarray(a, dtype=np.float32)
        elif a.dtype not in (np.float16, np.float32):
            raise TypeError(f"{ours}: GGUF writer handles float16/float32 only, got {a.dtype}")
        a = np.ascontiguousarray(a)
        typ = GGML_F16 if a.dtype == np.float16 else GGML_F32
        dims = tuple(reversed(a.shape))  # ggml order: innermost first
        infos.append(_gguf_str(gname) + struct.pack("<I", len(dims)) +
                     b"".join(struct.pack("<Q", d) for d in dims) + struct.pack("<IQ", typ, off))
        blobs.append((off, a))
        off = (off + a.nbytes + alignment - 1) // alignment * alignment
    with open(path, "wb") as f:
        f.write(struct.pack("<IIQQ", GGUF_MAGIC, version, len(infos), len(kv)))
        for b in kv:
            f.write(b)
        for b in infos:
            f.write(b)
        pos = f.tell()
        data_start = (pos + alignment - 1) // alignment * alignment
        f.write(b"\0" * (data_start - pos))
        for o, a in blobs:
            f.seek(data_start + o)
            a.tofile(f)
        f.truncate(data_start + off)  # pads the last tensor up to the alignment


class _Cursor:
    def __init__(self, buf, path):
        self.b, self.p, self.path = buf, 0, path

    def take(self, n: int) -> bytes:
        if self.p + n > len(self.b):
            raise ValueError(f"{self.path}: truncated GGUF (wanted {n} bytes at {self.p})")
        out = bytes(self.b[self.p:self.p + n])
        self.p += n
        return out

    def scalar(self, fmt: str):
        return struct.unpack(fmt, self.take(struct.calcsize(fmt)))[0]

    def string(self) -> str:
        n = self.scalar("<Q")
        if n > (1 << 30):
            raise ValueError(f"{self.path}: absurd GGUF string length {n}")
        return self.take(n).decode("utf-8", errors="replace")

    def value(self, typ: int, count_only_strings: bool = False):
        if typ == T_STR:
            return self.string()
        if typ == T_ARR:
            etyp = self.scalar("<I")
            n = self.scalar("<Q")
            if etyp == T_STR and count_only_strings:
                for _ in range(n):
                    ln = self.scalar("<Q")
                    self.take(ln)
                return ("strings", n)
            if etyp in _SCALAR:
                sz = struct.calcsize(_SCALAR[etyp])
                raw = self.take(sz * n)
                return np.frombuffer(raw, dtype=np.dtype(_SCALAR[etyp][1:]).newbyteorder("<"))
            return [self.value(etyp) for _ in range(n)]
        if typ not in _SCALAR:
            raise ValueError(f"{self.path}: unknown GGUF metadata type {typ}")
        return self.scalar(_SCALAR[typ])


def read_gguf(path: str) -> Tuple[ModelConfig, Dict[str, np.ndarray], Dict[str, object]]:
    """Parse a llama-architecture F32/F16 GGUF (v2 or v3) into (config, stacked tensors, metadata).

    Returned matrices are memory-mapped views stacked per layer on demand (one copy per tensor
    family); dtype is preserved.  Unlike the reference (src/loader.cpp:325-331) the context length
    is NOT clamped to 16384, and ``general.alignment`` is honoured (the reference assumes 32,
    src/gguf.cpp:262-264).
    """
    raw = np.memmap(path, dtype=np.uint8, mode="r")
    cur = _Cursor(raw, path)
    if cur.scalar("<I") != GGUF_MAGIC:
        raise ValueError(f"{path}: bad GGUF magic")
    version = cur.scalar("<I")
    if version not in (2, 3):
        raise ValueError(f"{path}: unsupported GGUF version {version} (need 2 or 3)")
    n_tensors, n_kv = cur.scalar("<Q"), cur.scalar("<Q")
    if n_tensors > 1 << 20 or n_kv > 1 << 20:
        raise ValueError(f"{path}: implausible GGUF counts ({n_tensors} tensors, {n_kv} keys)")
    meta: Dict[str, object] = {}
    for _ in range(n_kv):
        key = cur.string()
        typ = cur.scalar("<I")
        meta[key] = cur.value(typ, count_only_strings=True)
    infos = []
    for _ in range(n_tensors):
        name = cur.string()
        nd = cur.scalar("<I")
        if not 1 <= nd <= 4:
            raise ValueError(f"{path}: tensor {name} has {nd} dims")
        dims = [cur.scalar("<Q") for _ in range(nd)]
        typ, off = cur.scalar("<I"), cur.scalar("<Q")
        infos.append((name, dims, typ, off))
    align = int(meta.get("general.alignment", 32))
    data_start = (cur.p + align - 1) // align * align

    arch = meta.get("general.architecture")
    if not isinstance(arch, str):
        raise ValueError(f"{path}: missing general.architecture")

    def need(k):
        if f"{arch}.{k}" not in meta:
            raise ValueError(f"{path}: missing {arch}.{k}")
        return meta[f"{arch}.{k}"]

    toks = meta.get("tokenizer.ggml.tokens")
    if not (isinstance(toks, tuple) and toks[0] == "strings" and toks[1] > 0):
        raise ValueError(f"{path}: missing tokenizer.ggml.tokens")
    n_heads = int(need("attention.head_count"))
    c = ModelConfig(int(need("embedding_length")), int(need("feed_forward_length")), int(need("block_count")),
                    n_heads, int(meta.get(f"{arch}.attention.head_count_kv", n_heads)), int(toks[1]),
                    int(need("context_length")), float(meta.get(f"{arch}.rope.freq_base", 10000.0)))

    by_name = {}
    for name, dims, typ, off in infos:
        if typ not in (GGML_F32, GGML_F16):
            raise ValueError(f"{path}: tensor {name} has unsupported ggml type {typ} (F32/F16 only)")
        dt = np.float16 if typ == GGML_F16 else np.float32
        n = int(np.prod(dims))
        start = data_start + off
        if start + n * np.dtype(dt).itemsize > raw.size:
            raise ValueError(f"{path}: tensor {name} runs past the end of the file")
        by_name[name] = np.frombuffer(raw, dtype=dt, count=n, offset=start).reshape(tuple(reversed(dims)))

    tied = "output.weight" not in by_name
    shapes = tensor_shapes(c, tied)
    out: Dict[str, np.ndarray] = {}
    for gname, ours, layer in _gguf_tensor_names(c, tied):
        if gname not in by_name:
            raise ValueError(f"{path}: missing tensor {gname}")
        a = by_name[gname]
        want = shapes[ours] if layer is None else shapes[ours][1:]
        if a.shape != want:
            raise ValueError(f"{path}: tensor {gname} has shape {a.shape}, expected {want}")
        if layer is None:
            out[ours] = a
        else:
            if ours not in out:
                out[ours] = np.empty(shapes[ours], dtype=a.dtype)
            out[ours][layer] = a
    return c, out, meta


def is_gguf(path: str) -> bool:
    with open(path, "rb") as f:
        b = f.read(4)
    return len(b) == 4 and struct.unpack("<I", b)[0] == GGUF_MAGIC


def load_model(path: str) -> Tuple[ModelConfig, Dict[str, np.ndarray]]:
    """Either format, like ``main.cpp``'s ``is_gguf_file`` dispatch (src/main.cpp:44-113)."""
    if is_gguf(path):
        c, t, _ = read_gguf(path)
        return c, t
    return read_llama2c_bin(path)
