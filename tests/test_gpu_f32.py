"""f32 GEMM / Linear forward and backward on the GPU (3xTF32 on tcgen05) against the
CPU oracle (f64 accumulate, one rounding).  Tolerance is the one the task states:
max-abs error <= 1e-5 * sqrt(K) * max|A| * max|B|."""
import numpy as np
import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gemm_path")]


def tol(K, A, B):
    return 1e-5 * np.sqrt(K) * float(np.abs(A).max()) * float(np.abs(B).max())


@pytest.mark.parametrize("ta,tb,M,N,K", [
    (0, 0, 2, 2, 2), (0, 1, 64, 256, 784), (0, 0, 64, 10, 256), (1, 0, 256, 784, 64),
    (0, 1, 130, 70, 33), (1, 1, 300, 200, 100), (0, 1, 512, 512, 2048), (0, 0, 128, 384, 1000),
])
def test_gemm_f32(dev, orc, ta, tb, M, N, K):
    rng = np.random.default_rng(M + 2 * N + 3 * K + ta + 2 * tb)
    A = rng.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    B = rng.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    dA, dB = dev.to_device(A), dev.to_device(B)
    dC = dev.zeros((M, N), np.float32)
    dev.gemm_f32(ta, tb, M, N, K, dA, dB, dC)
    assert dev.check_status() == 0
    ref = orc.matmul_f32(A, B, bool(ta), bool(tb))
    err = np.abs(dC.numpy() - ref).max()
    assert err <= tol(K, A, B), f"max abs err {err} > {tol(K, A, B)}"
    for b in (dA, dB, dC):
        b.free()


def test_matmul_identity_kat(dev):
    """la/la_test.v:30-37: I . B == B exactly."""
    a = np.array([[1.0, 0], [0.0, 1]], np.float32)
    b = np.array([[4.0, 1], [2.0, 2]], np.float32)
    dA, dB, dC = dev.to_device(a), dev.to_device(b), dev.zeros((2, 2), np.float32)
    dev.gemm_f32(0, 0, 2, 2, 2, dA, dB, dC)
    assert np.array_equal(dC.numpy(), b)


def test_linear_kat_from_reference_session_test(dev, orc):
    """autograd_cuda/device_session_test.v:25-48 and :60-80 (values in f32)."""
    x = np.array([[1.0, 2.0, 3.0]], np.float32)
    w = np.array([[0.1, 0.2, 0.3], [0.4, 0.5, 0.6]], np.float32)
    b = np.array([0.01, 0.02], np.float32)
    dx, dw, db = dev.to_device(x), dev.to_device(w), dev.to_device(b)
    dy = dev.zeros((1, 2), np.float32)
    dev.linear_fwd_f32(dx, dw, db, dy, 1, 2, 3)
    assert np.allclose(dy.numpy(), [[1.41, 3.22]], atol=1e-6)
    g = np.array([[1.0, 0.5]], np.float32)
    dg = dev.to_device(g)
    ddx, ddw, ddb = dev.zeros((1, 3)), dev.zeros((2, 3)), dev.zeros((2,))
    dev.linear_bwd_f32(dg, dx, dw, ddx, ddw, ddb, 1, 2, 3)
    rdx, rdw, rdb = orc.linear_bwd_f32(g, x, w)
    assert np.allclose(ddx.numpy(), rdx, atol=1e-6)
    assert np.allclose(ddw.numpy(), rdw, atol=1e-6)
    assert np.allclose(ddb.numpy(), rdb.ravel(), atol=1e-6)


@pytest.mark.parametrize("M,N,K,relu", [(64, 256, 784, True), (64, 10, 256, False),
                                        (300, 130, 90, True), (1024, 512, 512, True),
                                        # few output features, many inputs: the streaming kernels of linear_narrow.cu
                                        (256, 10, 16384, False), (37, 16, 2048, True), (5, 1, 4100, False),
                                        (130, 3, 6148, True)])
def test_linear_fwd_bwd(dev, orc, M, N, K, relu):
    rng = np.random.default_rng(M + N + K)
    X = rng.random((M, K), dtype=np.float32)
    W = (rng.uniform(-1, 1, (N, K)) * np.sqrt(6.0 / K)).astype(np.float32)
    b = (rng.standard_normal(N) * 0.1).astype(np.float32)
    G = rng.standard_normal((M, N)).astype(np.float32)
    dX, dW_, db_, dG = (dev.to_device(a) for a in (X, W, b, G))
    dY, dPre = dev.zeros((M, N)), dev.zeros((M, N))
    dev.linear_fwd_f32(dX, dW_, db_, dY, M, N, K, relu, dPre if relu else None)
    assert dev.check_status() == 0
    pre = orc.linear_fwd_f32(X, W, b)
    ref = orc.relu_f32(pre) if relu else pre
    t = tol(K, X, W)
    assert np.abs(dY.numpy() - ref).max() <= t
    if relu:
        assert np.abs(dPre.numpy() - pre).max() <= t
    gdx, gdw, gdb = dev.zeros((M, K)), dev.zeros((N, K)), dev.zeros((N,))
    dev.linear_bwd_f32(dG, dX, dW_, gdx, gdw, gdb, M, N, K)
    assert dev.check_status() == 0
    rdx, rdw, rdb = orc.linear_bwd_f32(G, X, W)
    assert np.abs(gdx.numpy() - rdx).max() <= tol(N, G, W)
    assert np.abs(gdw.numpy() - rdw).max() <= tol(M, G, X)
    assert np.abs(gdb.numpy() - rdb.ravel()).max() <= tol(M, G, np.ones(1))


def test_gemm_f32_large_against_blas(dev, orc):
    """4096-wide layer at batch 2048: reference recipe with OpenBLAS dgemm."""
    M, N, K = 2048, 4096, 4096
    rng = np.random.default_rng(4)
    X = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.uniform(-1, 1, (N, K)) * np.sqrt(6.0 / K)).astype(np.float32)
    dX, dW_ = dev.to_device(X), dev.to_device(W)
    dY = dev.zeros((M, N))
    dev.linear_fwd_f32(dX, dW_, None, dY, M, N, K)
    assert dev.check_status() == 0
    ref = orc.matmul_f32_blas(X, W, tb=True)
    err = np.abs(dY.numpy() - ref).max()
    assert err <= tol(K, X, W), f"{err} vs {tol(K, X, W)}"


@pytest.mark.parametrize("M,N,K", [(256, 512, 384), (640, 256, 1024), (200, 100, 36), (130, 102, 38)])
def test_linear_planes_handed_from_producer_to_consumer(dev, orc, M, N, K):
    """vtlb_linear_fwd_f32_planes / _bwd_f32_planes: the planes a product leaves are the TF32 split of
    its stored result (rows and transposed), results are the same bit for bit with and without planes,
    and the ReLU backward applied in the dX product equals vtlb_relu_bwd_f32 on the unmasked dX.
    The last shape (row pitches that are no multiple of 16 bytes, so no TMA stores) takes the route
    with separate passes."""
    dev.set_small_gemm_limit(0.0)  # every product on the tensor-core path
    try:
        rng = np.random.default_rng(M + N + K)
        X = rng.standard_normal((M, K)).astype(np.float32)
        W = (rng.standard_normal((N, K)) * 0.1).astype(np.float32)
        b = (rng.standard_normal(N) * 0.1).astype(np.float32)
        G = rng.standard_normal((M, N)).astype(np.float32)
        Pre = rng.standard_normal((M, K)).astype(np.float32)   # pre-activation of the layer below
        dX_, dW_, db_, dG_, dPre = (dev.to_device(a) for a in (X, W, b, G, Pre))
        # plain calls
        Y0, pre0 = dev.zeros((M, N)), dev.zeros((M, N))
        dev.linear_fwd_f32(dX_, dW_, db_, Y0, M, N, K, relu=True, pre=pre0)
        gx0, gw0, gb0 = dev.zeros((M, K)), dev.zeros((N, K)), dev.zeros(N)
        dev.linear_bwd_f32(dG_, dX_, dW_, gx0, gw0, gb0, M, N, K)
        masked0 = dev.zeros((M, K))
        dev.relu_bwd_f32(gx0, dPre, masked0, M * K)
        # forward with planes in and out
        x_rows, x_cols = dev.planes(M, K), dev.planes(K, M)
        dev.split_planes_f32(dX_, M, K, rows=x_rows, cols=x_cols)
        hi, lo = orc.tf32_split(X)
        assert np.array_equal(x_rows.numpy()[0], hi) and np.array_equal(x_rows.numpy()[1], lo)
        assert np.array_equal(x_cols.numpy()[0], hi.T) and np.array_equal(x_cols.numpy()[1], lo.T)
        Y1, pre1 = dev.zeros((M, N)), dev.zeros((M, N))
        y_rows, y_cols = dev.planes(M, N), dev.planes(N, M)
        dev.linear_fwd_f32_planes(dX_, dW_, db_, Y1, M, N, K, relu=True, pre=pre1, x_rows=x_rows, y_rows=y_rows,
                                  y_cols=y_cols)
        assert np.array_equal(Y1.numpy().view(np.uint32), Y0.numpy().view(np.uint32))
        assert np.array_equal(pre1.numpy().view(np.uint32), pre0.numpy().view(np.uint32))
        hi, lo = orc.tf32_split(Y1.numpy())
        assert np.array_equal(y_rows.numpy()[0], hi) and np.array_equal(y_rows.numpy()[1], lo)
        assert np.array_equal(y_cols.numpy()[0], hi.T) and np.array_equal(y_cols.numpy()[1], lo.T)
        # backward with planes in, mask and planes out
        g_rows, g_cols = dev.planes(M, N), dev.planes(N, M)
        dev.split_planes_f32(dG_, M, N, rows=g_rows, cols=g_cols)
        gx1, gw1, gb1 = dev.zeros((M, K)), dev.zeros((N, K)), dev.zeros(N)
        dx_rows, dx_cols = dev.planes(M, K), dev.planes(K, M)
        dev.linear_bwd_f32_planes(dG_, dX_, dW_, gx1, gw1, gb1, M, N, K, g_rows=g_rows, g_cols=g_cols, x_cols=x_cols,
                                  relu_mask_src=dPre, dx_rows=dx_rows, dx_cols=dx_cols)
        assert dev.check_status() == 0
        assert np.array_equal(gw1.numpy().view(np.uint32), gw0.numpy().view(np.uint32))
        assert np.array_equal(gb1.numpy().view(np.uint32), gb0.numpy().view(np.uint32))
        assert np.array_equal(gx1.numpy().view(np.uint32), masked0.numpy().view(np.uint32))
        hi, lo = orc.tf32_split(gx1.numpy())
        assert np.array_equal(dx_rows.numpy()[0], hi) and np.array_equal(dx_rows.numpy()[1], lo)
        assert np.array_equal(dx_cols.numpy()[0], hi.T) and np.array_equal(dx_cols.numpy()[1], lo.T)
        # mask without planes, planes without mask
        gx2 = dev.zeros((M, K))
        dev.linear_bwd_f32_planes(dG_, dX_, dW_, gx2, None, None, M, N, K, relu_mask_src=dPre)
        assert np.array_equal(gx2.numpy().view(np.uint32), masked0.numpy().view(np.uint32))
        gx3 = dev.zeros((M, K))
        dev.linear_bwd_f32_planes(dG_, dX_, dW_, gx3, None, None, M, N, K, dx_rows=dx_rows)
        assert np.array_equal(gx3.numpy().view(np.uint32), gx0.numpy().view(np.uint32))
        assert np.array_equal(dx_rows.numpy()[0], orc.tf32_split(gx0.numpy())[0])
    finally:
        dev.set_small_gemm_limit(1.4e8)


@pytest.mark.parametrize("M,N,K", [(64, 10, 256), (33, 7, 100), (256, 10, 16384), (48, 256, 784), (32, 1024, 64)])
def test_relu_mask_on_the_cuda_core_routes(dev, M, N, K):
    """The ReLU backward handed to a small dX product (in the CUDA-core kernel's epilogue, cluster
    exchange and partial-buffer variants alike) and to a narrow layer (a pass behind the streaming
    kernel) equals vtlb_relu_bwd_f32 on the unmasked dX, bit for bit; zeros in the cache pass."""
    dev.set_small_gemm_limit(1.4e8)
    rng = np.random.default_rng(M * 7 + N + K)
    X = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((N, K)) * 0.1).astype(np.float32)
    G = rng.standard_normal((M, N)).astype(np.float32)
    Pre = rng.standard_normal((M, K)).astype(np.float32)
    Pre[0, :3] = [0.0, -0.0, -1.0]
    dX_, dW_, dG_, dPre = (dev.to_device(a) for a in (X, W, G, Pre))
    gx0, gw0, gb0 = dev.zeros((M, K)), dev.zeros((N, K)), dev.zeros(N)
    dev.linear_bwd_f32(dG_, dX_, dW_, gx0, gw0, gb0, M, N, K)
    want = dev.zeros((M, K))
    dev.relu_bwd_f32(gx0, dPre, want, M * K)
    gx1, gw1, gb1 = dev.to_device(np.full((M, K), 3.0, np.float32)), dev.zeros((N, K)), dev.zeros(N)
    dev.linear_bwd_f32_planes(dG_, dX_, dW_, gx1, gw1, gb1, M, N, K, relu_mask_src=dPre)
    assert dev.check_status() == 0
    assert np.array_equal(gx1.numpy().view(np.uint32), want.numpy().view(np.uint32))
    assert np.array_equal(gw1.numpy().view(np.uint32), gw0.numpy().view(np.uint32))
    assert np.array_equal(gb1.numpy().view(np.uint32), gb0.numpy().view(np.uint32))
    assert gx1.numpy()[0, 2] == 0.0 and gx1.numpy()[0, 0] == gx0.numpy()[0, 0]


def test_linear_planes_argument_errors(dev):
    from vtl_b200.capi import VtlbError, EINVAL
    x, w, y = dev.zeros((8, 8)), dev.zeros((8, 8)), dev.zeros((8, 8))
    pl = dev.planes(8, 8)
    with pytest.raises(VtlbError) as e:   # a mask or dX planes make no sense without dX
        dev.linear_bwd_f32_planes(y, x, w, None, y, None, 8, 8, 8, relu_mask_src=x)
    assert e.value.code == EINVAL
    with pytest.raises(VtlbError):
        dev.linear_bwd_f32_planes(y, x, w, None, y, None, 8, 8, 8, dx_rows=pl)
    pl.c.lo = None
    with pytest.raises(VtlbError):
        dev.linear_fwd_f32_planes(x, w, None, y, 8, 8, 8, x_rows=pl)
    assert dev.plane_ld(5) == 8 and dev.plane_ld(4096) == 4096
    dev.set_small_gemm_limit(1.4e8)  # small products run on CUDA cores, which read no planes
    assert not dev.f32_planes_worthwhile(64, 10, 256) and dev.f32_planes_worthwhile(8192, 4096, 4096)
