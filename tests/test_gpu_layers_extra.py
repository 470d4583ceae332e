"""Softmax, average pooling, BatchNorm1D and the SGD / RMSProp steps against the CPU restatement of
the reference's arithmetic.  Element-wise f32 / f64 formulas are bit-exact; results that go through
exp() or through long f64 sums (summed in slices on the device, in sequence on the CPU) are rounded
from f64 to f32 at the end and may differ in the last f32 bit: tolerance 1 ulp, stated per test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def ulp_diff(a, b):
    a, b = np.asarray(a, np.float32), np.asarray(b, np.float32)
    ia, ib = a.view(np.int32).astype(np.int64), b.view(np.int32).astype(np.int64)
    ia = np.where(ia < 0, -(ia & 0x7fffffff), ia)
    ib = np.where(ib < 0, -(ib & 0x7fffffff), ib)
    return int(np.abs(ia - ib).max()) if a.size else 0


@pytest.mark.parametrize("rows,n", [(1, 1), (3, 10), (256, 10), (1000, 1000), (7, 33)])
def test_softmax_forward_and_backward(dev, orc, rows, n):
    rng = np.random.default_rng(rows * 31 + n)
    x = (rng.standard_normal((rows, n)) * 3).astype(np.float32)
    g = rng.standard_normal((rows, n)).astype(np.float32)
    dx_, dg, dy, ddx = dev.to_device(x), dev.to_device(g), dev.zeros((rows, n)), dev.zeros((rows, n))
    dev.softmax_fwd_f32(dx_, rows, n, dy)
    dev.softmax_bwd_f32(dg, dx_, rows, n, ddx)
    y, dx = dy.numpy(), ddx.numpy()
    ref_y, ref_dx = orc.softmax_fwd_f32(x), orc.softmax_bwd_f32(g, x)
    assert ulp_diff(y, ref_y) <= 1                       # exp() of two maths libraries, then one rounding
    assert np.allclose(y.sum(axis=1), 1.0, atol=1e-5)
    # backward: f32 sums of n products of values that may differ in their last bit
    tol = 4 * n * np.finfo(np.float32).eps * max(1.0, float(np.abs(g).max()))
    assert np.abs(dx - ref_dx).max() <= tol
    for b in (dx_, dg, dy, ddx):
        b.free()


@pytest.mark.parametrize("shape,k,p,s", [((2, 3, 8, 8), (2, 2), (0, 0), (2, 2)), ((1, 1, 4, 4), (2, 2), (0, 0), (2, 2)),
                                         ((3, 2, 9, 7), (3, 3), (1, 1), (2, 1)), ((2, 4, 5, 5), (3, 2), (1, 0), (1, 1))])
def test_avgpool(dev, orc, shape, k, p, s):
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape).astype(np.float32)
    B, C, H, W = shape
    ref = orc.avgpool2d_fwd_f32(x, k, p, s)
    g = rng.standard_normal(ref.shape).astype(np.float32)
    dx_, dy, dg, ddx = dev.to_device(x), dev.zeros(ref.shape), dev.to_device(g), dev.zeros(shape)
    dev.avgpool2d_fwd_f32(dx_, dy, B, C, H, W, k[0], k[1], p[0], p[1], s[0], s[1])
    dev.avgpool2d_bwd_f32(dg, ddx, B, C, H, W, k[0], k[1], p[0], p[1], s[0], s[1])
    assert np.array_equal(dy.numpy().view(np.uint32), ref.view(np.uint32))
    assert np.array_equal(ddx.numpy().view(np.uint32), orc.avgpool2d_bwd_f32(g, shape, k, p, s).view(np.uint32))
    for b in (dx_, dy, dg, ddx):
        b.free()


def test_avgpool_known_answer(dev):
    """4x4 input 0..15, 2x2 windows: means 2.5, 4.5, 10.5, 12.5; backward spreads g/4."""
    x = np.arange(16, dtype=np.float32).reshape(1, 1, 4, 4)
    dx_, dy = dev.to_device(x), dev.zeros((1, 1, 2, 2))
    dev.avgpool2d_fwd_f32(dx_, dy, 1, 1, 4, 4, 2, 2, 0, 0, 2, 2)
    assert dy.numpy().reshape(-1).tolist() == [2.5, 4.5, 10.5, 12.5]
    dg, ddx = dev.to_device(np.array([4, 8, 12, 16], np.float32)), dev.zeros((1, 1, 4, 4))
    dev.avgpool2d_bwd_f32(dg, ddx, 1, 1, 4, 4, 2, 2, 0, 0, 2, 2)
    assert ddx.numpy().reshape(4, 4).tolist() == [[1, 1, 2, 2], [1, 1, 2, 2], [3, 3, 4, 4], [3, 3, 4, 4]]
    for b in (dx_, dy, dg, ddx):
        b.free()


def test_global_avgpool(dev, orc):
    rng = np.random.default_rng(3)
    shape = (5, 7, 6, 9)
    x = rng.standard_normal(shape).astype(np.float32)
    g = rng.standard_normal((5, 7, 1, 1)).astype(np.float32)
    dx_, dy, dg, ddx = dev.to_device(x), dev.zeros((5, 7, 1, 1)), dev.to_device(g), dev.zeros(shape)
    dev.global_avgpool2d_fwd_f32(dx_, dy, *shape)
    dev.global_avgpool2d_bwd_f32(dg, ddx, *shape)
    assert ulp_diff(dy.numpy(), orc.global_avgpool2d_fwd_f32(x)) <= 1   # lane-parallel f64 sum vs sequential
    assert np.array_equal(ddx.numpy().view(np.uint32), orc.global_avgpool2d_bwd_f32(g, shape).view(np.uint32))
    for b in (dx_, dy, dg, ddx):
        b.free()


@pytest.mark.parametrize("B,F", [(4, 3), (64, 256), (1000, 33), (8192, 512)])
def test_batchnorm1d(dev, orc, B, F):
    rng = np.random.default_rng(B + F)
    x = (rng.standard_normal((B, F)) * 2 + 0.5).astype(np.float32)
    gamma = rng.uniform(0.5, 1.5, F).astype(np.float32)
    beta = rng.standard_normal(F).astype(np.float32)
    rm0, rv0 = rng.standard_normal(F).astype(np.float32), rng.uniform(0.5, 2, F).astype(np.float32)
    g = rng.standard_normal((B, F)).astype(np.float32)
    d = {k: dev.to_device(v) for k, v in dict(x=x, gamma=gamma, beta=beta, rm=rm0, rv=rv0, g=g).items()}
    dy, dmean, dvar = dev.zeros((B, F)), dev.zeros(F), dev.zeros(F)
    dev.batchnorm1d_train_f32(d["x"], B, F, d["gamma"], d["beta"], 1e-5, dy, dmean, dvar, d["rm"], d["rv"], 0.1)
    y, mean, var, rm, rv = orc.batchnorm1d_train_f32(x, gamma, beta, 1e-5, rm0, rv0, 0.1)
    # sliced f64 sums on the device, sequential on the CPU, both rounded to f32 at the end
    assert ulp_diff(dmean.numpy(), mean) <= 1 and ulp_diff(dvar.numpy(), var) <= 1
    assert ulp_diff(d["rm"].numpy(), rm) <= 1 and ulp_diff(d["rv"].numpy(), rv) <= 1
    assert np.abs(dy.numpy() - y).max() <= 2e-6 * max(1.0, float(np.abs(y).max()))
    # inference path: f32 element-wise, bit-exact
    dyi = dev.zeros((B, F))
    drm, drv = dev.to_device(rm), dev.to_device(rv)
    dev.batchnorm1d_infer_f32(d["x"], B, F, d["gamma"], d["beta"], drm, drv, 1e-5, dyi)
    assert np.array_equal(dyi.numpy().view(np.uint32), orc.batchnorm1d_infer_f32(x, gamma, beta, rm, rv, 1e-5).view(np.uint32))
    # backward with the oracle's (f32-rounded) batch statistics
    dm, dv = dev.to_device(mean), dev.to_device(var)
    ddx, ddg, ddb = dev.zeros((B, F)), dev.zeros(F), dev.zeros(F)
    dev.batchnorm1d_bwd_f32(d["g"], d["x"], B, F, d["gamma"], dm, dv, 1e-5, ddx, ddg, ddb)
    rdx, rdg, rdb = orc.batchnorm1d_bwd_f32(g, x, gamma, mean, var, 1e-5)
    assert np.abs(ddx.numpy() - rdx).max() <= 2e-6 * max(1.0, float(np.abs(rdx).max()))
    scale = float(np.sqrt(B)) * 4
    assert np.abs(ddg.numpy() - rdg).max() <= 1e-6 * scale * max(1.0, float(np.abs(rdg).max()) / scale)
    assert ulp_diff(ddb.numpy(), rdb) <= 1
    for b in list(d.values()) + [dy, dmean, dvar, dyi, drm, drv, dm, dv, ddx, ddg, ddb]:
        b.free()


def test_batchnorm_known_answer(dev):
    """x = [[0,1,2],[3,4,5],[6,7,8],[9,10,11]]: means 4.5, 5.5, 6.5; biased variances 11.25."""
    x = np.arange(12, dtype=np.float32).reshape(4, 3)
    dx_, dg, db = dev.to_device(x), dev.to_device(np.ones(3, np.float32)), dev.to_device(np.zeros(3, np.float32))
    dy, dm, dv = dev.zeros((4, 3)), dev.zeros(3), dev.zeros(3)
    dev.batchnorm1d_train_f32(dx_, 4, 3, dg, db, 0.0, dy, dm, dv)
    assert dm.numpy().tolist() == [4.5, 5.5, 6.5] and dv.numpy().tolist() == [11.25] * 3
    want = (x - x.mean(0)) / np.sqrt(11.25)
    assert np.allclose(dy.numpy(), want, atol=1e-6)
    for b in (dx_, dg, db, dy, dm, dv):
        b.free()


@pytest.mark.parametrize("n", [1, 5, 4096, 100003])
def test_sgd_and_rmsprop_steps_bit_exact(dev, orc, n):
    rng = np.random.default_rng(n)
    g = rng.standard_normal(n).astype(np.float32)
    th = rng.standard_normal(n).astype(np.float32)
    sq = rng.uniform(0, 1, n).astype(np.float32)
    dg, dth = dev.to_device(g), dev.to_device(th)
    dev.sgd_step_f32(dev.adam_table([(dg, dth, None, None, n)]), 0.05, zero_grad=True)
    assert np.array_equal(dth.numpy().view(np.uint32), orc.sgd_step_f32(g, th, 0.05).view(np.uint32))
    assert not dg.numpy().any()
    dg2, dth2, dsq = dev.to_device(g), dev.to_device(th), dev.to_device(sq)
    for wd in (0.0, 0.01):
        ref_th, ref_sq = orc.rmsprop_step_f32(g, dth2.numpy(), dsq.numpy(), 1e-3, 0.99, 1e-8, wd)
        dev.rmsprop_step_f32(dev.adam_table([(dg2, dth2, None, dsq, n)]), 1e-3, 0.99, 1e-8, wd, zero_grad=False)
        assert np.array_equal(dth2.numpy().view(np.uint32), ref_th.view(np.uint32))
        assert np.array_equal(dsq.numpy().view(np.uint32), ref_sq.view(np.uint32))
    for b in (dg, dth, dg2, dth2, dsq):
        b.free()


def test_argument_errors(dev):
    from vtl_b200.capi import VtlbError
    d = dev.zeros(16)
    with pytest.raises(VtlbError, match="bad geometry"):
        dev.avgpool2d_fwd_f32(d, d, 1, 1, 4, 4, 0, 2, 0, 0, 2, 2)
    with pytest.raises(VtlbError, match="empty output"):
        dev.avgpool2d_fwd_f32(d, d, 1, 1, 2, 2, 3, 3, 0, 0, 1, 1)
    with pytest.raises(VtlbError, match="bad shape"):
        dev.batchnorm1d_infer_f32(d, 0, 4, d, d, d, d, 1e-5, d)
    with pytest.raises(VtlbError, match="null pointer"):
        dev.rmsprop_step_f32(dev.adam_table([(d, d, None, None, 16)]), 1e-3, 0.99, 1e-8, 0.0)
    d.free()
