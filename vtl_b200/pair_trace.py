"""Where the cycles of the INT8 CTA-pair GEMM go: a tuning aid, not part of the product path.

    python -m vtl_b200.build --trace          # builds vtl_b200/libvtlb200_trace.so (no GPU needed)
    python -m vtl_b200.pair_trace [M N K]     # on a B200; default 4096 4096 4096

The trace library is the normal one with int8.cu compiled with -DVTLB_PAIR_TRACE: every role of
every CTA (TMA producer, MMA issuer, epilogue warp 2) accumulates the SM cycles it spends in each of
its waits, and the MMA thread notes when it has issued the last MMA of each of its work units.  The
counters cost a few clock reads per K block, so times under the trace are a few per cent longer than
the product's; compare shares, not absolutes.
"""
from __future__ import annotations

import ctypes
import os
import sys

import numpy as np

from . import capi
from .build import TRACE_LIB


def main(argv):
    M, N, K = (int(a) for a in argv[:3]) if len(argv) >= 3 else (4096, 4096, 4096)
    if not os.path.exists(TRACE_LIB):
        raise SystemExit(f"{TRACE_LIB} is missing: run `python -m vtl_b200.build --trace` first")
    capi.LIB_PATH = TRACE_LIB
    dev = capi.Device(0)
    dev.lib.vtlb_debug_pair_trace.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    rng = np.random.default_rng(0)
    dA = dev.to_device(rng.integers(-127, 128, size=(M, K), dtype=np.int8))
    dW = dev.to_device(rng.integers(-127, 128, size=(N, K), dtype=np.int8))
    dSa = dev.to_device(np.full(M, 0.01, np.float32))
    dSw = dev.to_device(np.full(N, 0.01, np.float32))
    db = dev.to_device(np.zeros(N, np.float32))
    dY = dev.zeros((M, N))

    def run():
        dev.linear_i8_fwd(dA, dSa, dW, dSw, db, dY, M, N, K, True)

    for _ in range(5):
        run()
    e0, e1 = dev.event(), dev.event()
    dev.record(e0)
    run()
    dev.record(e1)
    us = dev.elapsed_ms(e0, e1) * 1e3
    out = np.zeros(160 * 24, np.int64)
    dev.lib.vtlb_debug_pair_trace(dev.h, out.ctypes.data_as(ctypes.c_void_p))  # clears the phase counters
    run()
    rc = dev.lib.vtlb_debug_pair_trace(dev.h, out.ctypes.data_as(ctypes.c_void_p))
    if rc != 0 or dev.check_status() != 0:
        raise SystemExit(f"trace failed: rc={rc} status={dev.check_status()}")
    ep = out[160 * 16:].reshape(160, 8)
    tr = out[:160 * 16].reshape(160, 16)
    ncta = int(np.count_nonzero(tr[:, 5]))
    tr, ep = tr[:ncta], ep[:ncta]
    lead = tr[0::2]

    def st(x):
        return f"min {int(x.min()):7d}  median {int(np.median(x)):7d}  max {int(x.max()):7d}"

    print(f"fused INT8 linear M={M} N={N} K={K}: {us:.1f} us for one launch under the trace, {ncta} CTAs")
    print("cycles per CTA (SM clock):")
    print("  TMA producer  total         ", st(tr[:, 0]))
    print("                waiting: empty", st(tr[:, 1]))
    print("  MMA issuer    total         ", st(lead[:, 2]))
    print("                waiting: full ", st(lead[:, 3]))
    print("                waiting: tmem ", st(lead[:, 4]))
    print("  epilogue w2   total         ", st(tr[:, 5]))
    print("                waiting: accum", st(tr[:, 6]))
    n = np.maximum(ep[:, 4], 1)
    print("epilogue warp 2, cycles per 32x32 chunk (median over CTAs): "
          f"tmem load {int(np.median(ep[:, 0] // n))}, transform {int(np.median(ep[:, 1] // n))}, "
          f"wait for the staging tile {int(np.median(ep[:, 2] // n))}, stage + issue store {int(np.median(ep[:, 3] // n))}")
    print("cycle at which the MMA thread had issued the last MMA of its i-th unit:")
    for u in range(8):
        col = lead[:, 8 + u]
        if col.max() > 0:
            print(f"  unit {u}: {int(np.count_nonzero(col)):3d} pairs ", st(col[col > 0]))


if __name__ == "__main__":
    main(sys.argv[1:])
