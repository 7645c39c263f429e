"""CPU tests: the plain-C restatement (oracle/lpp_oracle.c) is pinned against
(a) the known-answer vectors of the reference's own unit tests (src/runtests.cpp:87-306),
(b) golden vectors produced by the compiled reference (tests/golden/make_golden.py),
(c) the compiled reference itself, bit for bit, where oracle/_ref is present."""
import numpy as np
import pytest

from lighterpp_b200 import synth

SETTINGS = [(0.0, 1.0), (0.0, 1.3), (1.0, 1.0), (0.8, 1.1)]


# ---- (a) known-answer tests of src/runtests.cpp -------------------------------------------------

def test_kat_matmul_square(oracle):  # runtests.cpp:87-103
    out = oracle.matmul([1, 2], [[1, 0], [0, 1]])
    assert np.allclose(out, [1.0, 2.0], atol=1e-4)


def test_kat_matmul_rectangular(oracle):  # runtests.cpp:105-126
    out = oracle.matmul([1, 2, 3], [[0.5, 0.5, 1.0], [2.0, 0.0, 1.0]])
    assert np.allclose(out, [4.5, 5.0], atol=1e-4)


def test_kat_rmsnorm(oracle):  # runtests.cpp:128-144
    out = oracle.rmsnorm([2, 2, 2, 2], [1, 1, 1, 1])
    assert np.allclose(out, 1.0, atol=1e-4)


def test_kat_rope(oracle):  # runtests.cpp:147-184: position 0 is the identity, position 1 rotates
    q = np.array([1, 0, 1, 0], dtype=np.float32)
    q0, k0 = oracle.rope(q, q, 0, 4, 10000.0)
    assert np.allclose(q0, q, atol=1e-4) and np.allclose(k0, q, atol=1e-4)
    q1, _ = oracle.rope(q, q, 1, 4, 10000.0)
    assert not np.allclose(q1, q, atol=1e-4)
    assert np.allclose(q1[:2], [np.cos(1.0), np.sin(1.0)], atol=1e-4)


def test_kat_softmax(oracle):  # runtests.cpp:256-283
    assert np.allclose(oracle.softmax([1, 2, 3]), [0.09003, 0.24473, 0.66524], atol=1e-4)


def test_kat_swiglu(oracle):  # runtests.cpp:285-306
    assert np.allclose(oracle.swiglu([1.0, -1.0], [2.0, 3.0]), [1.46211, -0.80682], atol=1e-4)


# ---- (b) golden vectors from the compiled reference ---------------------------------------------

def test_ops_match_golden(oracle, golden):
    x, w, g = golden["ops/x"], golden["ops/w"], golden["ops/g"]
    assert np.array_equal(oracle.matmul(x, w), golden["ops/matmul"])
    assert np.array_equal(oracle.rmsnorm(x, g), golden["ops/rmsnorm"])
    q, k = oracle.rope(x, x[:48], 7, 48, 10000.0)
    assert np.array_equal(q, golden["ops/rope_q"]) and np.array_equal(k, golden["ops/rope_k"])
    q, k = oracle.rope(x, x[:32], 33000, 32, 500000.0)
    assert np.array_equal(q, golden["ops/rope_q_far"]) and np.array_equal(k, golden["ops/rope_k_far"])
    assert np.array_equal(oracle.softmax(x), golden["ops/softmax"])
    assert np.array_equal(oracle.swiglu(x, g), golden["ops/swiglu"])


@pytest.mark.parametrize("name", ["tiny-f32", "tiny-gqa-f16", "tiny-tp8-f16"])
def test_steps_match_golden(oracle, golden, name):
    c, dt, tied, seed, T = synth.named(name)
    m = oracle.model(c, synth.as_f32(T))
    toks = golden[f"{name}/tokens"]
    for pos, t in enumerate(toks):
        assert np.array_equal(m.step_logits(int(t), pos), golden[f"{name}/logits"][pos]), (name, pos)
    k, v = m.kv_cache()
    n = len(toks)
    assert np.array_equal(k[:, :, :n], golden[f"{name}/k"])
    assert np.array_equal(v[:, :, :n], golden[f"{name}/v"])
    assert not k[:, :, n:].any()  # nothing written beyond the steps taken


@pytest.mark.parametrize("name", ["tiny-f32", "tiny-gqa-f16", "tiny-tp8-f16"])
def test_sample_matches_golden(oracle, golden, name):
    logits = golden[f"{name}/logits"][-1]
    hist, rs = golden[f"{name}/history"], golden[f"{name}/r"]
    assert np.array_equal(oracle.rand_floats(1234, len(rs)), rs)  # libc rand() stream
    for si, (temp, pen) in enumerate(SETTINGS):
        for di, r in enumerate(rs):
            assert oracle.sample(logits, temp, pen, hist, float(r)) == golden[f"{name}/sample_ids"][si, di]


def test_kv_index_formula(oracle):
    # layer*(kv_dim*S) + head*(S*hs) + pos*hs + off  (src/scatter_kv.cu:15-16 == src/model.cpp:173)
    L, KVH, S, hs = 3, 4, 50, 16
    seen = set()
    for l in range(L):
        for h in range(KVH):
            for p in (0, 1, S - 1):
                for off in (0, hs - 1):
                    i = oracle.kv_index(l, h, p, off, KVH, hs, S)
                    assert i == l * (KVH * hs * S) + h * (S * hs) + p * hs + off
                    seen.add(i)
    assert len(seen) == L * KVH * 3 * 2 and max(seen) == L * KVH * S * hs - 1


# ---- (c) bit-for-bit against the compiled reference -----------------------------------------------

@pytest.mark.parametrize("name", ["tiny-f32", "tiny-gqa-f16"])
def test_restatement_equals_reference(oracle, reference, name):
    c, dt, tied, seed, T = synth.named(name)
    W = synth.as_f32(T)
    a, b = oracle.model(c, W), reference.model(c, W)
    rng = np.random.default_rng(5)
    toks = rng.integers(0, c.vocab_size, size=20)
    for pos, t in enumerate(toks):
        la, lb = a.step_logits(int(t), pos), b.step_logits(int(t), pos)
        assert np.array_equal(la, lb)
    for temp, pen in SETTINGS:
        for seed_ in (1, 2, 3):
            r = reference.rand_floats(seed_, 1)[0]
            assert oracle.sample(la, temp, pen, toks, float(r)) == reference.sample(lb, temp, pen, toks, seed=seed_)


def test_reference_forward_entry_point(oracle, reference):
    """forward() itself (src/model.cpp:342-384) = step logits + sample with the rand() stream."""
    c, dt, tied, seed, T = synth.named("tiny-f32")
    W = synth.as_f32(T)
    a, b = oracle.model(c, W), reference.model(c, W)
    rs = oracle.rand_floats(77, 6)
    reference.srand(77)
    tok = 5
    hist = [5]
    for pos in range(6):
        nxt_ref = b.forward(tok, pos, 0.9, 1.1, hist)
        nxt = oracle.sample(a.step_logits(tok, pos), 0.9, 1.1, hist, float(rs[pos]))
        assert nxt == nxt_ref
        tok = nxt
        hist.append(tok)
