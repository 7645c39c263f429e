"""GPU test of lpp_op_sample_static, the sampler entry point that allocates nothing.

Hosts that have given away all their device memory up front, or that are in the middle of a global-mode
stream capture, cannot let a library call the allocator; for them the sampler's scratch sits in a fixed
array inside the library.  This file calls that entry point through the C ABI and checks that it picks
exactly the token lpp_op_sample picks, on two calls in a row (the second must not see anything the first
left in the shared scratch), and that it refuses sizes beyond its built-in capacity.  The file name sorts
last so that a run stopping at the first failure has already executed every other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from lighterpp_b200 import engine as E
    lib = E.load_library()
    sig = [C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_void_p, C.c_int, C.c_float, C.c_void_p, C.c_void_p]
    lib.lpp_op_sample.argtypes = sig
    lib.lpp_op_sample_static.argtypes = sig
    return torch, lib


def _call(torch, fn, logits, temperature, penalty, hist, r):
    d_logits = torch.from_numpy(logits.copy()).cuda()  # both entry points modify the logits in place
    d_hist = torch.from_numpy(hist).cuda()
    out = torch.full((1,), -7, dtype=torch.int32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    st = fn(C.c_void_p(d_logits.data_ptr()), logits.size, temperature, penalty, C.c_void_p(d_hist.data_ptr()), hist.size,
            r, C.c_void_p(out.data_ptr()), stream)
    torch.cuda.synchronize()
    return st, int(out.item()), d_logits.cpu().numpy()


@pytest.mark.parametrize("V", [1000, 32000, 128256, 262144])
def test_static_scratch_sampler_matches_allocating_one(env, V):
    torch, lib = env
    rng = np.random.default_rng(V + 1)
    # two calls in a row with different inputs: long history then short, categorical then argmax; the largest
    # vocabulary runs at the entry point's built-in capacity (262144 logits, 4096 history entries)
    cases = [
        (rng.standard_normal(V).astype(np.float32), 0.8, 1.1,
         rng.integers(0, V, 4096 if V == 262144 else 64).astype(np.int32), 0.37),
        (rng.standard_normal(V).astype(np.float32) * 2, 0.0, 1.3, rng.integers(0, V, 5).astype(np.int32), 0.0),
        (rng.standard_normal(V).astype(np.float32), 1.0, 1.0, rng.integers(0, V, 1).astype(np.int32), 0.93),
    ]
    for logits, temperature, penalty, hist, r in cases:
        st_a, tok_a, lg_a = _call(torch, lib.lpp_op_sample_static, logits, temperature, penalty, hist, r)
        st_b, tok_b, lg_b = _call(torch, lib.lpp_op_sample, logits, temperature, penalty, hist, r)
        assert st_a == 0 and st_b == 0
        assert 0 <= tok_a < V
        assert tok_a == tok_b                      # same kernel, same arithmetic: identical token
        assert np.array_equal(lg_a, lg_b)          # and the same in-place effect on the logits


def test_static_scratch_sampler_leaves_device_memory_alone(env):
    """After its first call on the device the entry point allocates nothing: free device memory and the default
    memory pool's reservation are the same before and after a run of calls on pre-allocated buffers."""
    torch, lib = env
    V = 32000
    rng = np.random.default_rng(5)
    d_logits = torch.from_numpy(rng.standard_normal(V).astype(np.float32)).cuda()
    keep = d_logits.clone()
    d_hist = torch.from_numpy(rng.integers(0, V, 64).astype(np.int32)).cuda()
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def call(r):
        d_logits.copy_(keep)
        return lib.lpp_op_sample_static(C.c_void_p(d_logits.data_ptr()), V, 0.8, 1.1, C.c_void_p(d_hist.data_ptr()), 64, r,
                                        C.c_void_p(out.data_ptr()), stream)

    assert call(0.5) == 0  # the first call per device resolves the scratch address
    torch.cuda.synchronize()
    rt = C.CDLL("libcudart.so.12")
    pool = C.c_void_p()
    assert rt.cudaDeviceGetDefaultMemPool(C.byref(pool), torch.cuda.current_device()) == 0

    def reserved():
        v = C.c_uint64(0)
        assert rt.cudaMemPoolGetAttribute(pool, 5, C.byref(v)) == 0  # cudaMemPoolAttrReservedMemCurrent
        return v.value

    free0, res0 = torch.cuda.mem_get_info()[0], reserved()
    toks = []
    for r in (0.1, 0.37, 0.93):
        assert call(r) == 0
        torch.cuda.synchronize()
        toks.append(int(out.item()))
    assert torch.cuda.mem_get_info()[0] == free0 and reserved() == res0
    assert all(0 <= t < V for t in toks)


def test_static_scratch_sampler_rejects_oversize(env):
    torch, lib = env
    lib.lpp_last_error.restype = C.c_char_p
    buf = torch.zeros(8, device="cuda")
    out = torch.zeros(1, dtype=torch.int32, device="cuda")
    st = lib.lpp_op_sample_static(C.c_void_p(buf.data_ptr()), 262145, 1.0, 1.0, None, 0, 0.5, C.c_void_p(out.data_ptr()),
                                  None)
    assert st == 6 and b"262144" in lib.lpp_last_error()  # LPP_ERR_TOO_LARGE, nothing launched
    st = lib.lpp_op_sample_static(C.c_void_p(buf.data_ptr()), 8, 1.0, 1.5, C.c_void_p(out.data_ptr()), 5000, 0.5,
                                  C.c_void_p(out.data_ptr()), None)
    assert st == 6
    st = lib.lpp_op_sample_static(None, 8, 1.0, 1.0, None, 0, 0.5, C.c_void_p(out.data_ptr()), None)
    assert st == 1
