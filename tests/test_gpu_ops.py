"""GPU tests of the stand-alone operator entry points (the host wrappers of src/kernels.cuh:24-36) through
the C ABI, on the shapes and input patterns of the reference's own CUDA-vs-CPU tests
(src/runtests.cpp:313-875) plus seeded random cases, against the CPU oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def T():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch


def dev(T, a):
    return T.from_numpy(np.ascontiguousarray(a)).cuda()


def test_gemv_f32_runtests_pattern(T, oracle):  # runtests.cpp:313-383
    from lighterpp_b200 import ops
    n, d = 256, 512
    x = (0.1 * (np.arange(d) % 10)).astype(np.float32)
    w = (0.01 * (np.arange(n * d) % 100)).astype(np.float32).reshape(n, d)
    out = T.zeros(n, device="cuda")
    ops.cuda_gemv(out, dev(T, x), dev(T, w), n, d, ops.WEIGHT_FP32)
    assert np.abs(out.cpu().numpy() - oracle.matmul(x, w)).max() < 1e-3  # is_close_gpu, runtests.cpp:83-85


def test_gemv_f16_runtests_pattern(T, oracle):  # runtests.cpp:385-469
    from lighterpp_b200 import ops
    n, d = 256, 512
    x = (0.1 * (np.arange(d) % 10)).astype(np.float32)
    w = (0.01 * (np.arange(n * d) % 100)).astype(np.float32).reshape(n, d)
    w16 = T.empty((n, d), dtype=T.float16, device="cuda")
    ops.cuda_convert_f32_to_f16(w16, dev(T, w), n * d)
    assert np.array_equal(w16.cpu().numpy(), w.astype(np.float16))
    out = T.zeros(n, device="cuda")
    ops.cuda_gemv(out, dev(T, x), w16, n, d, ops.WEIGHT_FP16)
    ref = oracle.matmul(x, w)
    assert np.all(np.abs(out.cpu().numpy() - ref) <= 0.01 * np.abs(ref) + 1e-4)
    # against the FP16-rounded weights the result is FP32-accurate (x is not rounded to half)
    ref16 = oracle.matmul(x, w.astype(np.float16).astype(np.float32))
    assert np.abs(out.cpu().numpy() - ref16).max() < 2e-4 * np.abs(ref16).max()


@pytest.mark.parametrize("n,d,dt", [(2, 8, "f16"), (6, 4, "f32"), (7, 13, "f32"), (33, 40, "f16"), (4096, 2048, "f16"),
                                    (300, 14336, "f16")])
def test_gemv_shapes(T, oracle, n, d, dt):
    from lighterpp_b200 import ops
    rng = np.random.default_rng(n * 131 + d)
    x = rng.standard_normal(d).astype(np.float32)
    w = (rng.standard_normal((n, d)) * 0.05).astype(np.float16 if dt == "f16" else np.float32)
    out = T.zeros(n, device="cuda")
    ops.cuda_gemv(out, dev(T, x), dev(T, w), n, d, ops.WEIGHT_FP16 if dt == "f16" else ops.WEIGHT_FP32)
    ref = oracle.matmul(x, w.astype(np.float32))
    assert np.abs(out.cpu().numpy() - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())


def test_rmsnorm(T, oracle):  # runtests.cpp:471-520
    from lighterpp_b200 import ops
    n = 256
    x = (0.01 * (np.arange(n) % 100) + 0.5).astype(np.float32)
    w = (1.0 + 0.001 * np.arange(n)).astype(np.float32)
    out = T.zeros(n, device="cuda")
    ops.cuda_rmsnorm(out, dev(T, x), dev(T, w), n)
    assert np.abs(out.cpu().numpy() - oracle.rmsnorm(x, w)).max() < 1e-5


def test_rope(T, oracle):  # runtests.cpp:522-579 (dim 128, head size 64, pos 5) plus a far position
    from lighterpp_b200 import ops
    for pos, base in ((5, 10000.0), (1500, 500000.0)):
        q = (0.01 * np.arange(128)).astype(np.float32)
        k = (0.02 * np.arange(128)).astype(np.float32)
        dq, dk = dev(T, q), dev(T, k)
        ops.cuda_rope(dq, dk, pos, 128, 128, 64, base)
        rq, rk = oracle.rope(q, k, pos, 64, base)
        assert np.abs(dq.cpu().numpy() - rq).max() < 1e-3 and np.abs(dk.cpu().numpy() - rk).max() < 1e-3


def test_swiglu_residual_scale_softmax(T, oracle):  # runtests.cpp:581-797
    from lighterpp_b200 import ops
    n = 256
    h1 = (0.1 * (np.arange(n) % 20) - 1.0).astype(np.float32)
    h3 = (0.05 * (np.arange(n) % 10) + 0.5).astype(np.float32)
    out = T.zeros(n, device="cuda")
    ops.cuda_swiglu(out, dev(T, h1), dev(T, h3), n)
    assert np.abs(out.cpu().numpy() - oracle.swiglu(h1, h3)).max() < 1e-5
    a, b = h1, h3
    ops.cuda_residual_add(out, dev(T, a), dev(T, b), n)
    assert np.array_equal(out.cpu().numpy(), a + b)
    heads, t, stride = 4, 32, 64
    att = np.zeros((heads, stride), np.float32)
    att[:, :t] = (0.1 * (np.arange(heads * t) % 17)).reshape(heads, t)
    d = dev(T, att)
    ops.cuda_scale_multihead(d, 0.125, heads, t, stride)
    assert np.allclose(d.cpu().numpy()[:, :t], att[:, :t] * 0.125)
    assert not d.cpu().numpy()[:, t:].any()
    ops.cuda_softmax_multihead(d, d, heads, t, stride)
    got = d.cpu().numpy()
    for h in range(heads):
        assert np.abs(got[h, :t] - oracle.softmax(att[h, :t] * np.float32(0.125))).max() < 1e-6


def test_scatter_multihead_gemv_aggregation(T, oracle):  # runtests.cpp:799-875 + GQA
    from lighterpp_b200 import ops
    L, KVH, H, hs, S = 2, 2, 4, 16, 8
    rng = np.random.default_rng(3)
    kc = T.zeros(L * KVH * S * hs, dtype=T.float16, device="cuda")
    vc = T.zeros_like(kc)
    ks = rng.standard_normal((S, KVH * hs)).astype(np.float32)
    vs = rng.standard_normal((S, KVH * hs)).astype(np.float32)
    layer = 1
    for pos in range(S):
        ops.cuda_scatter_kv(kc, vc, dev(T, ks[pos]), dev(T, vs[pos]), layer, pos, KVH, hs, S)
    hk = kc.cpu().numpy().reshape(L, KVH, S, hs)
    assert not hk[0].any()
    for pos in range(S):
        for h in range(KVH):
            i0 = oracle.kv_index(layer, h, pos, 0, KVH, hs, S)
            assert np.array_equal(kc.cpu().numpy()[i0:i0 + hs], ks[pos, h * hs:(h + 1) * hs].astype(np.float16))
    q = rng.standard_normal(H * hs).astype(np.float32)
    att = T.zeros((H, S), device="cuda")
    ops.cuda_multihead_gemv(att, dev(T, q), kc, layer, S - 1, H, KVH, hs, S)
    k16 = ks.astype(np.float16).astype(np.float32)
    for h in range(H):
        kv = h // (H // KVH)
        ref = k16[:, kv * hs:(kv + 1) * hs] @ q[h * hs:(h + 1) * hs]
        assert np.abs(att.cpu().numpy()[h] - ref).max() < 1e-4
    probs = np.full((H, S), 1.0 / S, np.float32)
    out = T.zeros(H * hs, device="cuda")
    v_layer = vc[layer * KVH * S * hs:]
    ops.cuda_aggregation_multihead(out, v_layer, dev(T, probs), H, S, hs, H // KVH, S)
    v16 = vs.astype(np.float16).astype(np.float32)
    for h in range(H):
        kv = h // (H // KVH)
        ref = probs[h] @ v16[:, kv * hs:(kv + 1) * hs]
        assert np.abs(out.cpu().numpy()[h * hs:(h + 1) * hs] - ref).max() < 1e-4


def test_rope_scatter_fused_equals_separate(T):
    from lighterpp_b200 import ops
    rng = np.random.default_rng(8)
    dim, KVH, hs, S, layer, pos = 128, 2, 32, 16, 1, 9
    q = rng.standard_normal(dim).astype(np.float32)
    k = rng.standard_normal(KVH * hs).astype(np.float32)
    v = rng.standard_normal(KVH * hs).astype(np.float32)
    n = 2 * KVH * S * hs
    kc1, vc1 = T.zeros(n, dtype=T.float16, device="cuda"), T.zeros(n, dtype=T.float16, device="cuda")
    kc2, vc2 = T.zeros_like(kc1), T.zeros_like(vc1)
    q1, k1 = dev(T, q), dev(T, k)
    ops.cuda_rope(q1, k1, pos, dim, KVH * hs, hs, 10000.0)
    ops.cuda_scatter_kv(kc1, vc1, k1, dev(T, v), layer, pos, KVH, hs, S)
    q2 = dev(T, q)
    ops.cuda_rope_scatter(q2, dev(T, k), dev(T, v), kc2, vc2, layer, pos, dim, KVH, hs, S, 10000.0)
    assert T.equal(q1, q2) and T.equal(kc1, kc2) and T.equal(vc1, vc2)


@pytest.mark.parametrize("V", [320, 32000, 128256])
def test_cuda_sample_wrapper(T, oracle, V):
    from lighterpp_b200 import ops
    rng = np.random.default_rng(V)
    lg = rng.standard_normal(V).astype(np.float32)
    hist = np.array([1, 5, 5, V - 1, 7], dtype=np.int32)
    out = T.zeros(1, dtype=T.int32, device="cuda")
    for temp, pen in ((0.0, 1.0), (0.0, 1.5)):
        ops.cuda_sample(dev(T, lg), V, temp, pen, dev(T, hist), len(hist), 0.3, out)
        assert int(out.item()) == oracle.sample(lg, temp, pen, hist, 0.3)
