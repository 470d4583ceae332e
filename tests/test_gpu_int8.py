"""INT8 quantised linear path on the GPU against the CPU oracle: codes, scales and
int32 accumulators must be bit-exact; the dequantised output is bit-exact by
construction (checked as such)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _quant_gpu(dev, A):
    M, K = A.shape
    ld = dev.i8_ld(K)
    dA = dev.to_device(A)
    dQ = dev.zeros((M, ld), np.int8)
    dS = dev.empty((M,), np.float32)
    dev.quant_rows_i8(dA, M, K, dQ, dS)
    q = dQ.numpy()[:, :K]
    s = dS.numpy()
    dA.free()
    return dQ, dS, q, s


@pytest.mark.parametrize("M,K", [(1, 16), (3, 100), (64, 784), (257, 4096), (33, 4100)])
def test_quant_rows_bit_exact(dev, orc, M, K):
    rng = np.random.default_rng(100 + M + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    A[0, :] = 0.0  # an all-zero row: scale 0, codes 0
    if M > 2:
        A[2, 0] = 1e30  # a huge outlier
    dQ, dS, q, s = _quant_gpu(dev, A)
    q_ref, s_ref = orc.quant_rows_i8(A)
    assert np.array_equal(q, q_ref)
    assert np.array_equal(s.view(np.uint32), s_ref.view(np.uint32))
    dQ.free(); dS.free()


def test_quant_rows_with_given_amax(dev, orc):
    rng = np.random.default_rng(7)
    A = rng.standard_normal((40, 256)).astype(np.float32)
    amax = (np.abs(A).max(axis=1) * 1.5).astype(np.float32)
    dA, dM = dev.to_device(A), dev.to_device(amax)
    dQ, dS = dev.zeros((40, 256), np.int8), dev.empty((40,), np.float32)
    dev.quant_rows_i8(dA, 40, 256, dQ, dS, dM)
    q_ref, s_ref = orc.quant_rows_i8_with_amax(A, amax)
    assert np.array_equal(dQ.numpy(), q_ref)
    assert np.array_equal(dS.numpy().view(np.uint32), s_ref.view(np.uint32))
    dAm = dev.empty((40,), np.float32)
    dev.row_absmax_f32(dA, 40, 256, dAm)
    assert np.array_equal(dAm.numpy(), np.abs(A).max(axis=1))
    for b in (dA, dM, dQ, dS, dAm):
        b.free()


def _codes(rng, rows, K, ld):
    q = rng.integers(-127, 128, size=(rows, K), dtype=np.int8)
    buf = rng.integers(-128, 128, size=(rows, ld), dtype=np.int8)  # padding holds garbage on purpose
    buf[:, :K] = q
    return q, buf


SHAPES = [
    (1, 64, 128), (2, 1000, 4100), (5, 100, 48), (16, 4096, 4096),   # dp4a path (M = 1), few-row kernel
    (17, 64, 32), (128, 256, 128), (128, 64, 4096),        # one tile, each tile width
    (200, 328, 400), (129, 257, 144),                      # ragged M, N, K
    # few rows: swapped-operand kernel, every row-count class, K cut over clusters of 1, 2 and 4
    (7, 512, 520), (20, 4100, 1024), (33, 1000, 8192), (64, 4096, 4096), (100, 130, 272),
    (128, 18944, 256), (128, 4096, 4096),
    (48, 640, 1152),                                       # 9 K blocks over 4 CTAs: the last range is empty
    (512, 1024, 512), (1024, 4096, 1024),
    # more 256 x 256 tiles than CTA pairs with a short final wave: its tiles are cut along K
    # between two pairs (90 tiles and 256 tiles on 74 pairs)
    (2500, 2100, 1100), (4096, 4096, 1024), (2304, 2302, 1024),
]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_i8_i32_bit_exact(dev, orc, M, N, K):
    rng = np.random.default_rng(M * 7 + N * 3 + K)
    ld = dev.i8_ld(K)
    a, abuf = _codes(rng, M, K, ld)
    w, wbuf = _codes(rng, N, K, ld)
    dA, dW = dev.to_device(abuf), dev.to_device(wbuf)
    dC = dev.zeros((M, N), np.int32)
    dev.gemm_i8_i32(dA, dW, M, N, K, dC)
    assert dev.check_status() == 0
    got = dC.numpy()
    ref = orc.gemm_i8_i32(a, w)
    assert np.array_equal(got, ref), f"{np.count_nonzero(got != ref)} of {got.size} accumulators differ"
    for b in (dA, dW, dC):
        b.free()


@pytest.mark.parametrize("M,N,K,relu,bias", [
    (1, 256, 512, True, True), (16, 300, 128, False, True),
    (9, 4096, 4096, True, True), (40, 1002, 1152, False, True), (128, 4096, 2048, True, False),  # few-row kernel
    (128, 256, 256, True, True), (300, 500, 272, True, False), (512, 512, 1024, False, True),
    (2304, 2300, 1024, True, True),  # K-split final wave through the fused epilogue
])
def test_linear_i8_fwd_matches_oracle(dev, orc, M, N, K, relu, bias):
    rng = np.random.default_rng(M + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(N) * 0.01).astype(np.float32) if bias else None
    wq_ref, sw_ref = orc.quant_rows_i8(W)
    dQw, dSw, wq, sw = _quant_gpu(dev, W)
    assert np.array_equal(wq, wq_ref)
    dQa, dSa, _, _ = _quant_gpu(dev, A)
    db = dev.to_device(b) if bias else None
    dY = dev.zeros((M, N), np.float32)
    dev.linear_i8_fwd(dQa, dSa, dQw, dSw, db, dY, M, N, K, relu)
    assert dev.check_status() == 0
    ref = orc.linear_i8_fwd(A, wq_ref, sw_ref, b, relu)
    got = dY.numpy()
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32)), \
        f"max abs diff {np.abs(got - ref).max()}"
    for buf in (dQw, dSw, dQa, dSa, dY):
        buf.free()
    if db:
        db.free()


def test_config2_full_size_properties(dev, orc):
    """M=N=K=4096 (the benchmark configuration): too large for the scalar oracle in
    seconds, so check (a) a random sample of rows against the oracle bit-exactly and
    (b) linearity in int32: gemm(A, W) + gemm(A2, W) == gemm(A + A2, W) for small codes."""
    M = N = K = 4096
    rng = np.random.default_rng(2)
    a = rng.integers(-60, 61, size=(M, K), dtype=np.int8)
    a2 = rng.integers(-60, 61, size=(M, K), dtype=np.int8)
    w = rng.integers(-127, 128, size=(N, K), dtype=np.int8)
    dW = dev.to_device(w)
    outs = []
    for mat in (a, a2, (a + a2).astype(np.int8)):
        dA = dev.to_device(mat)
        dC = dev.zeros((M, N), np.int32)
        dev.gemm_i8_i32(dA, dW, M, N, K, dC)
        assert dev.check_status() == 0
        outs.append(dC.numpy())
        dA.free(); dC.free()
    assert np.array_equal(outs[0] + outs[1], outs[2])
    rows = rng.choice(M, size=24, replace=False)
    ref = orc.gemm_i8_i32(a[rows], w)
    assert np.array_equal(outs[0][rows], ref)
    dW.free()


def test_int8_argument_errors(dev):
    from vtl_b200.capi import VtlbError, EINVAL
    d = dev.zeros((16, 16), np.int8)
    c = dev.zeros((16, 16), np.int32)
    with pytest.raises(VtlbError) as e:
        dev.gemm_i8_i32(d, d, 16, 16, 0, c)
    assert e.value.code == EINVAL
    with pytest.raises(VtlbError):
        dev.gemm_i8_i32(d.ptr + 1, d, 64, 16, 16, c)  # misaligned operand
    dev.gemm_i8_i32(d, d, 0, 16, 16, c)  # empty M is a no-op
    d.free(); c.free()


@pytest.mark.parametrize("M,N,K,relu", [
    (2, 300, 256, False),            # dp4a path: the maxima come from a pass over Y
    (24, 1024, 1024, False),         # few-row kernel: likewise
    (200, 328, 400, True),           # single-CTA kernel, TMA-store epilogue
    (129, 258, 144, False),          # N % 4 != 0: direct stores
    (2304, 2300, 1024, False),       # CTA pairs with K-split tiles, negative outputs
    (1024, 4096, 512, True),
])
def test_linear_i8_fwd_amax_returns_the_row_maxima_of_its_output(dev, orc, M, N, K, relu):
    rng = np.random.default_rng(M * 3 + N + K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    b = (rng.standard_normal(N) * 0.01).astype(np.float32)
    dQw, dSw, wq, sw = _quant_gpu(dev, W)
    dQa, dSa, _, _ = _quant_gpu(dev, A)
    db, dY = dev.to_device(b), dev.zeros((M, N), np.float32)
    dmax = dev.to_device(np.full(M, 7.0, np.float32))  # stale contents must not survive
    dev.linear_i8_fwd_amax(dQa, 1, dSa, dQw, dSw, db, dY, M, N, K, relu, dmax)
    assert dev.check_status() == 0
    ref = orc.linear_i8_fwd(A, wq, sw, b, relu)
    got = dY.numpy()
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(dmax.numpy().view(np.uint32), np.abs(ref).max(axis=1).view(np.uint32))
    for buf in (dQw, dSw, dQa, dSa, db, dY, dmax):
        buf.free()


def test_int8_issue_yardstick(dev):
    """The no-load INT8 MMA loop runs, leaves the status clean and reports a rate of the order of the
    device's INT8 tensor throughput (nominally 4.5 POPS dense; well above any real GEMM here)."""
    tops = dev.int8_issue_yardstick(4000)
    assert dev.check_status() == 0
    assert 1500.0 < tops < 6000.0, tops
    from vtl_b200.capi import VtlbError
    with pytest.raises(VtlbError):
        dev.int8_issue_yardstick(0)
