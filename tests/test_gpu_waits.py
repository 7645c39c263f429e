"""Bounded device-side waits: a wait that cannot be satisfied must run out, the kernel must return
normally, the host call must fail with LPP_ERR_DEVICE_STATUS (5) and the context must stay usable.
Nothing here traps, faults or spins without a limit: the waits are the product's own, with the limit
shortened through lpp_config (wait_ms / tp_wait_ms)."""
import ctypes as C
import time

import numpy as np
import pytest

from lighterpp_b200 import synth

pytestmark = pytest.mark.gpu

DEVICE_STATUS = 5


@pytest.fixture(scope="module")
def E():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from lighterpp_b200 import engine
    return engine


def test_wait_on_a_barrier_nobody_arrives_on_runs_out(E):
    c, dt, tied, seed, T = synth.named("tiny-gqa-f16")
    eng = E.Engine(c, dt, "f16", wait_ms=5)
    eng.load_weights(T)
    first = eng.forward(3, 0)
    eng.lib.lpp_debug_wait_probe.argtypes = [C.c_void_p]
    t0 = time.perf_counter()
    status = eng.lib.lpp_debug_wait_probe(eng.h)
    dt_s = time.perf_counter() - t0
    assert status == DEVICE_STATUS, status
    assert b"barrier timeout" in eng.lib.lpp_last_error()
    assert dt_s < 2.0, dt_s  # 5 ms of SM clocks, not the default limit and not forever
    # the context and the engine are still usable: the next step clears the status and gives the same token
    assert eng.forward(3, 0) == first
    eng.close()


def test_wait_on_an_absent_tensor_parallel_peer_runs_out(E):
    """Rank 0 of a two-rank group runs alone (its stores to rank 1 go to a scratch buffer, nobody fills rank 1's
    slot of its receive areas): the first GEMV that consumes an exchange gives up after tp_wait_ms, every later
    kernel of the step sees the status bit and does not spin again, and lpp_step returns status 5."""
    c, dt, tied, seed, T = synth.named("tiny-tp8-f16")
    eng = E.Engine(c, dt, "f16", tp_rank=0, tp_size=2, flags=E.FLAG_TP_LOCAL, tp_wait_ms=20)
    eng.lib.lpp_debug_tp_absent_peers.argtypes = [C.c_void_p]
    assert eng.lib.lpp_debug_tp_absent_peers(eng.h) == 0
    eng.load_weights(T)
    for _ in range(2):  # the status is cleared per call: the second call waits (bounded) again
        t0 = time.perf_counter()
        with pytest.raises(E.LppError) as ei:
            eng.forward(3, 0)
        dt_s = time.perf_counter() - t0
        assert ei.value.status == DEVICE_STATUS
        # one 20 ms wait per step, not one per consuming kernel (2 layers -> 5 consumers) and not seconds
        assert dt_s < 1.0, dt_s
    eng.close()
    # a fresh single-GPU engine on the same context works
    c2, dt2, _, _, T2 = synth.named("tiny-gqa-f16")
    ok = E.Engine(c2, dt2, "f16")
    ok.load_weights(T2)
    assert 0 <= ok.forward(1, 0) < c2.vocab_size
    ok.close()


def test_tp_local_engine_needs_its_peers(E):
    c, dt, tied, seed, T = synth.named("tiny-tp8-f16")
    eng = E.Engine(c, dt, "f16", tp_rank=0, tp_size=2, flags=E.FLAG_TP_LOCAL)
    with pytest.raises(E.LppError) as ei:
        eng.load_weights(T)
    assert ei.value.status == 3 and "lpp_tp_connect" in str(ei.value)
    eng.close()
