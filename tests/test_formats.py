"""CPU tests for the model-file formats on either side of the path (llama2.c .bin, GGUF F32/F16)."""
import struct

import numpy as np
import pytest

from lighterpp_b200 import formats, synth


@pytest.mark.parametrize("name", ["tiny-f32", "tiny-gqa-f16", "tiny-tp8-f16"])
def test_gguf_roundtrip(tmp_path, name):
    c, dt, tied, seed, T = synth.named(name)
    p = str(tmp_path / "m.gguf")
    formats.write_gguf(p, c, T)
    assert formats.is_gguf(p)
    c2, T2, meta = formats.read_gguf(p)
    assert c2 == c and set(T2) == set(T)
    for k in T:
        assert T2[k].dtype == T[k].dtype and np.array_equal(T2[k], T[k]), k
    assert meta["general.architecture"] == "llama"


def test_bin_roundtrip(tmp_path):
    c, dt, tied, seed, T = synth.named("tiny-f32")
    p = str(tmp_path / "m.bin")
    formats.write_llama2c_bin(p, c, T)
    assert not formats.is_gguf(p)
    c2, T2 = formats.load_model(p)
    assert c2 == c
    for k in T:
        assert np.array_equal(T2[k], T[k]), k


def test_reference_loaders_accept_our_files(tmp_path, reference):
    """The unmodified reference loaders (src/loader.cpp, src/gguf.cpp) read what we write."""
    for name in ["tiny-f32", "tiny-gqa-f16"]:
        c, dt, tied, seed, T = synth.named(name)
        for ext, write in (("bin", formats.write_llama2c_bin), ("gguf", formats.write_gguf)):
            if ext == "bin" and dt != "f32":
                continue
            p = str(tmp_path / f"{name}.{ext}")
            write(p, c, T)
            m = reference.load(p)
            assert m.cfg == c
            direct = reference.model(c, synth.as_f32(T))
            assert np.array_equal(m.step_logits(3, 0), direct.step_logits(3, 0))


def test_gguf_v2_and_alignment(tmp_path):
    c, dt, tied, seed, T = synth.named("tiny-gqa-f16")
    p = str(tmp_path / "m.gguf")
    formats.write_gguf(p, c, T, version=2)
    assert formats.read_gguf(p)[0] == c


def test_malformed_files(tmp_path):
    c, dt, tied, seed, T = synth.named("tiny-f32")
    good = tmp_path / "good.gguf"
    formats.write_gguf(str(good), c, T)
    raw = good.read_bytes()
    cases = {
        "bad_magic": b"XXXX" + raw[4:],
        "bad_version": raw[:4] + struct.pack("<I", 7) + raw[8:],
        "truncated_header": raw[:20],
        "truncated_data": raw[:len(raw) - 4096],
    }
    for name, blob in cases.items():
        p = tmp_path / f"{name}.gguf"
        p.write_bytes(blob)
        with pytest.raises(ValueError):
            formats.read_gguf(str(p))
    # missing tensor
    T2 = dict(T)
    p = tmp_path / "short.bin"
    p.write_bytes(b"\0" * 10)
    with pytest.raises(ValueError):
        formats.read_llama2c_bin(str(p))
    formats.write_llama2c_bin(str(tmp_path / "ok.bin"), c, T2)
    blob = (tmp_path / "ok.bin").read_bytes()
    (tmp_path / "cut.bin").write_bytes(blob[:len(blob) // 2])
    with pytest.raises(ValueError):
        formats.read_llama2c_bin(str(tmp_path / "cut.bin"))


def test_synth_is_deterministic_per_tensor():
    c, dt, tied, seed = synth.SHAPES["tiny-gqa-f16"]
    a = synth.gen_tensor(c, "w1", seed, dt, layer=1)
    b = synth.gen_model(c, seed, dt, tied)["w1"][1]
    assert a.dtype == np.float16 and np.array_equal(a, b)
    assert abs(float(np.std(b.astype(np.float32))) - 0.02) < 2e-3
    assert np.all(synth.gen_model(c, seed, dt, tied)["rms_att"] == 1.0)
