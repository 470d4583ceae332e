"""Failure detection on the device side: a bounded wait that runs out is reported through the
status word as VTLB_ETIMEOUT, the kernel returns, and the context stays usable.  The wait is
made to run out by not arriving on its barrier (nothing faults, traps or spins unbounded)."""
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_bounded_wait_gives_up_and_reports_timeout(dev, orc):
    from vtl_b200 import capi
    assert dev.check_status() == 0
    # satisfied wait: nothing is reported
    dev.wait_probe(2_000_000, arrive=True)
    assert dev.check_status() == 0
    # a wait nobody satisfies, limit 2 ms: the kernel comes back on its own ...
    t0 = time.perf_counter()
    dev.wait_probe(2_000_000, arrive=False)
    with pytest.raises(capi.VtlbError) as ei:
        dev.check_status()
    assert time.perf_counter() - t0 < 1.0
    assert ei.value.code == capi.ETIMEOUT
    assert "wait ran out" in str(ei.value)
    # ... the status word was cleared by the read, and the context still computes correctly
    assert dev.check_status() == 0
    rng = np.random.default_rng(0)
    A = rng.standard_normal((200, 96)).astype(np.float32)
    B = rng.standard_normal((64, 96)).astype(np.float32)
    dA, dB, dC = dev.to_device(A), dev.to_device(B), dev.zeros((200, 64))
    dev.set_small_gemm_limit(0.0)  # the tcgen05 path, whose waits share the routine just tested
    dev.gemm_f32(False, True, 200, 64, 96, dA, dB, dC)
    dev.set_small_gemm_limit(1.4e8)
    assert dev.check_status() == 0
    ref = orc.matmul_f32(A, B, tb=True)
    assert np.abs(dC.numpy() - ref).max() <= 1e-5 * np.sqrt(96) * np.abs(A).max() * np.abs(B).max()


def test_wait_probe_rejects_long_limits(dev):
    from vtl_b200 import capi
    for bad in (0, 200_000_000):
        with pytest.raises(capi.VtlbError) as ei:
            dev.wait_probe(bad, arrive=False)
        assert ei.value.code == capi.EINVAL
