"""Conv2D forward/backward and max pooling on the GPU against the CPU oracle.  The oracle
accumulates in f32 in (ic,kh,kw) order as the reference does; the GPU runs the lowered 3xTF32
GEMM, so the comparison uses the stated bound 1e-5*sqrt(K)*max|A|*max|B| with K the
contraction length of each product."""
import json
import os

import numpy as np
import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.usefixtures("gemm_path")]
HERE = os.path.dirname(os.path.abspath(__file__))


def tol(K, A, B):
    return 1e-5 * np.sqrt(K) * float(np.abs(A).max()) * float(np.abs(B).max())


def run_conv(dev, x, w, b, pad, stride, relu=False):
    B, C, H, W = x.shape
    O, _, kh, kw = w.shape
    OH = (H + 2 * pad[0] - kh) // stride[0] + 1
    OW = (W + 2 * pad[1] - kw) // stride[1] + 1
    dx, dw = dev.to_device(x), dev.to_device(w)
    db = dev.to_device(b) if b is not None else None
    dy, dpre = dev.zeros((B, O, OH, OW)), dev.zeros((B, O, OH, OW))
    dev.conv2d_fwd_f32(dx, dw, db, dy, B, C, H, W, O, kh, kw, pad[0], pad[1], stride[0], stride[1], relu,
                       dpre if relu else None)
    assert dev.check_status() == 0
    return dy.numpy(), dpre.numpy()


def run_conv_bwd(dev, g, x, w, pad, stride):
    B, C, H, W = x.shape
    O, _, kh, kw = w.shape
    dg, dx, dw = dev.to_device(g), dev.to_device(x), dev.to_device(w)
    gdx, gdw, gdb = dev.zeros(x.shape), dev.zeros(w.shape), dev.zeros(O)
    dev.conv2d_bwd_f32(dg, dx, dw, gdx, gdw, gdb, B, C, H, W, O, kh, kw, pad[0], pad[1], stride[0], stride[1])
    assert dev.check_status() == 0
    return gdx.numpy(), gdw.numpy(), gdb.numpy()


def test_conv2d_reference_kat(dev):
    """nn/internal/conv2d_cuda_test.v:32-59, 85-122 (1x1x4x4 input 1..16, 3x3 kernel, pad 1)."""
    k = json.load(open(os.path.join(HERE, "golden", "reference_kats.json")))["conv2d_4x4"]
    x = np.array(k["input"], np.float32).reshape(1, 1, 4, 4)
    w = np.array(k["weight"], np.float32).reshape(1, 1, 3, 3)
    y, _ = run_conv(dev, x, w, np.zeros(1, np.float32), k["pad"], k["stride"])
    assert np.abs(y.reshape(4, 4) - np.array(k["forward"])).max() < k["tol_fwd"]
    g = np.array(k["grad_out"], np.float32).reshape(1, 1, 4, 4)
    dx, dw, db = run_conv_bwd(dev, g, x, w, k["pad"], k["stride"])
    assert np.abs(dx.reshape(4, 4) - np.array(k["d_input"])).max() < k["tol_bwd"]
    assert np.abs(dw.reshape(3, 3) - np.array(k["d_weight"])).max() < k["tol_bwd"]
    assert abs(float(db[0]) - k["d_bias"]) < k["tol_bwd"]


@pytest.mark.parametrize("B,C,H,W,O,k,pad,stride", [
    (2, 3, 32, 32, 32, 3, 1, 1),      # conv1 of the CNN configuration (small batch)
    (2, 32, 32, 32, 64, 3, 1, 1),     # conv2
    (3, 5, 9, 11, 7, 3, 0, 1),        # ragged everything, no padding
    (2, 4, 12, 10, 6, 2, 1, 2),       # even kernel, stride 2
    (1, 1, 4, 4, 1, 2, 0, 1),         # conv2d_cuda_test.v:7-19 shape case -> [1,1,3,3]
    (2, 6, 13, 13, 70, 5, 2, 1),      # 25 taps, more output channels than one 64-wide tile
    (1, 3, 7, 9, 4, 7, 3, 1),         # 49 taps: beyond the implicit GEMM's tap mask, lowered path
    (3, 2, 10, 8, 5, 3, 2, 3),        # stride 3: implicit forward, lowered input gradient
    (5, 16, 11, 6, 8, 1, 0, 1),       # 1x1 kernel
    (3, 64, 12, 8, 96, 3, 1, 1),      # slab kernel: two / three channel groups, two 64-wide output tiles
    (2, 32, 9, 8, 40, 5, 2, 1),       # slab kernel: 25 taps, one partly filled tile per image
    (2, 32, 10, 14, 32, 3, 0, 1),     # slab kernel forward without padding (input gradient: gathered)
    (5, 32, 33, 32, 64, 3, 1, 1),     # slab kernel: 11 tiles of 3 rows per image, the last one clipped
    (40, 3, 8, 8, 16, 3, 1, 1),       # weight gradient over pixels: CTAs start in the middle of images
    (7, 40, 6, 5, 130, 3, 1, 1),      # ... two channel groups (the second partly filled), three output blocks
    (9, 8, 5, 31, 9, 2, 0, 1),        # ... 2x2 window, 30-pixel rows that are no multiple of 4
    (2, 4, 6, 40, 6, 3, 1, 1),        # output rows longer than 32 pixels: the lowered weight gradient
])
def test_conv2d_fwd_bwd_vs_oracle(dev, orc, B, C, H, W, O, k, pad, stride):
    rng = np.random.default_rng(B * 100 + C * 10 + O)
    x = rng.standard_normal((B, C, H, W)).astype(np.float32)
    w = (rng.uniform(-1, 1, (O, C, k, k)) * np.sqrt(6.0 / (C * k * k))).astype(np.float32)
    b = (rng.standard_normal(O) * 0.1).astype(np.float32)
    y, pre = run_conv(dev, x, w, b, (pad, pad), (stride, stride), relu=True)
    ref = orc.conv2d_fwd_f32(x, w, b, pad=(pad, pad), stride=(stride, stride))
    Kc = C * k * k
    assert y.shape == ref.shape
    assert np.abs(pre - ref).max() <= tol(Kc, x, w)
    assert np.abs(y - orc.relu_f32(ref)).max() <= tol(Kc, x, w)
    g = rng.standard_normal(ref.shape).astype(np.float32)
    dx, dw, db = run_conv_bwd(dev, g, x, w, (pad, pad), (stride, stride))
    rdx, rdw, rdb = orc.conv2d_bwd_f32(g, x, w, pad=(pad, pad), stride=(stride, stride))
    Mc = B * ref.shape[2] * ref.shape[3]
    assert np.abs(dx - rdx).max() <= tol(O * k * k, g, w)
    assert np.abs(dw - rdw).max() <= tol(Mc, g, x)
    assert np.abs(db - rdb.ravel()).max() <= tol(Mc, g, np.ones(1))


def test_conv2d_split_k_path(dev, orc):
    """A batch large enough for the d_weight GEMM to split its contraction over CTAs."""
    rng = np.random.default_rng(9)
    B, C, H, W, O = 16, 8, 32, 32, 16
    x = rng.standard_normal((B, C, H, W)).astype(np.float32)
    w = (rng.standard_normal((O, C, 3, 3)) * 0.1).astype(np.float32)
    g = rng.standard_normal((B, O, H, W)).astype(np.float32)
    dx, dw, db = run_conv_bwd(dev, g, x, w, (1, 1), (1, 1))
    rdx, rdw, rdb = orc.conv2d_bwd_f32(g, x, w, pad=(1, 1), stride=(1, 1))
    assert np.abs(dw - rdw).max() <= tol(B * H * W, g, x)
    assert np.abs(dx - rdx).max() <= tol(O * 9, g, w)
    assert np.abs(db - rdb.ravel()).max() <= tol(B * H * W, g, np.ones(1))


@pytest.mark.parametrize("shape", [(2, 3, 6, 8), (4, 64, 32, 32), (1, 1, 2, 4), (3, 5, 10, 12)])
def test_maxpool2x2_backward_direct_and_with_relu(dev, orc, shape):
    """The tiling 2x2 window: dX written directly equals the scatter onto zeros bit for bit; with the
    cache of a ReLU in front of the pool it equals scatter followed by that ReLU's backward -- which
    zeroes where the cache is negative and lets the gradient pass where it is exactly zero."""
    rng = np.random.default_rng(sum(shape) + 1)
    pre = rng.standard_normal(shape).astype(np.float32)
    pre[0, 0, 0, :2] = -1.0
    pre[0, 0, 1, :2] = [-0.5, -2.0]  # a window that is negative throughout: its gradient must vanish
    pre[0, 0, 0, 2:4] = [0.0, -1.0]
    pre[0, 0, 1, 2:4] = [-3.0, -0.25]  # the winner of this window is an exact zero: the gradient passes
    x = orc.relu_f32(pre)
    ry, ridx = orc.maxpool2d_fwd_f32(x, (2, 2), (0, 0), (2, 2))
    B, C, H, W = shape
    dx = dev.to_device(x)
    dy, didx = dev.zeros(ry.shape), dev.zeros(ry.shape, np.int32)
    dev.maxpool2d_fwd_f32(dx, dy, didx, B, C, H, W, 2, 2, 0, 0, 2, 2)
    g = rng.standard_normal(ry.shape).astype(np.float32)
    dg = dev.to_device(g)
    out = dev.to_device(np.full(shape, 9.0, np.float32))  # stale contents must not survive
    dev.maxpool2x2_bwd_f32(dg, didx, None, out, B, C, H, W)
    scat = orc.maxpool2d_bwd_f32(g, ridx, shape)
    assert np.array_equal(out.numpy().view(np.uint32), scat.view(np.uint32))
    dpre = dev.to_device(pre)
    dev.maxpool2x2_bwd_f32(dg, didx, dpre, out, B, C, H, W)
    ref = orc.relu_bwd_f32(scat, pre)
    assert np.array_equal(out.numpy(), ref)
    assert not out.numpy()[0, 0, :2, :2].any()
    # relu(window) = [0, 0; 0, 0]: the first position wins, and its pre-activation is 0, not negative
    assert ridx[0, 0, 0, 1] == 2 and out.numpy()[0, 0, 0, 2] == g[0, 0, 0, 1] != 0.0
    from vtl_b200 import capi
    with pytest.raises(capi.VtlbError):
        dev.maxpool2x2_bwd_f32(dg, didx, None, out, B, C, H, W + 2)
    assert dev.check_status() == 0


@pytest.mark.parametrize("shape,kernel,pad,stride", [((2, 3, 6, 8), (2, 2), (0, 0), (2, 2)),
                                                      ((4, 64, 32, 32), (2, 2), (0, 0), (2, 2)),
                                                      ((2, 3, 5, 6), (2, 2), (0, 0), (2, 2)),   # general kernel
                                                      ((1, 2, 7, 7), (3, 3), (1, 1), (2, 2))])
def test_maxpool_bit_exact(dev, orc, shape, kernel, pad, stride):
    rng = np.random.default_rng(sum(shape))
    x = rng.standard_normal(shape).astype(np.float32)
    x[0, 0, 0, :2] = 5.0  # a tie inside the first window: the first maximum must win
    x[0, 0, 0, 3] = x[0, 0, 1, 2] = 7.0  # and one across the two rows of the second window
    ry, ridx = orc.maxpool2d_fwd_f32(x, kernel, pad, stride)
    dx = dev.to_device(x)
    dy, didx = dev.zeros(ry.shape), dev.zeros(ry.shape, np.int32)
    B, C, H, W = shape
    dev.maxpool2d_fwd_f32(dx, dy, didx, B, C, H, W, kernel[0], kernel[1], pad[0], pad[1], stride[0], stride[1])
    assert np.array_equal(dy.numpy(), ry)
    assert np.array_equal(didx.numpy(), ridx)
    g = rng.standard_normal(ry.shape).astype(np.float32)
    dg, dgx = dev.to_device(g), dev.zeros(shape)
    dev.maxpool2d_bwd_f32(dg, didx, dgx, g.size, x.size)
    ref = orc.maxpool2d_bwd_f32(g, ridx, shape)
    if stride[0] >= kernel[0]:
        assert np.array_equal(dgx.numpy(), ref)
    else:  # overlapping windows add in a different order
        assert np.abs(dgx.numpy() - ref).max() <= 1e-6


@pytest.mark.parametrize("B,C,H,W,O,k,pad,stride,dil", [
    (2, 3, 12, 11, 5, 3, (2, 2), (1, 1), (2, 2)),   # "same" output with dilation 2
    (3, 4, 13, 9, 6, 3, (1, 0), (2, 1), (2, 3)),    # different dilation per axis, stride 2 down the rows
    (1, 2, 7, 7, 3, 2, (0, 0), (1, 1), (3, 3)),     # 2x2 window spread over 4x4
    (2, 3, 8, 8, 4, 3, (1, 1), (1, 1), (1, 1)),     # dilation 1 through the same entry point
])
def test_conv2d_dilated_vs_oracle(dev, orc, B, C, H, W, O, k, pad, stride, dil):
    """Dilated windows (Conv2DConfig.dilation; conv2d_forward_cpu_f32.v:26-62, conv2d_backward_cpu_f32.v)."""
    rng = np.random.default_rng(B + C + H + O + dil[0])
    x = rng.standard_normal((B, C, H, W)).astype(np.float32)
    w = (rng.uniform(-1, 1, (O, C, k, k)) * np.sqrt(6.0 / (C * k * k))).astype(np.float32)
    b = (rng.standard_normal(O) * 0.1).astype(np.float32)
    ref = orc.conv2d_fwd_f32(x, w, b, pad=pad, stride=stride, dil=dil)
    _, _, OH, OW = ref.shape
    dx_, dw_, db_ = dev.to_device(x), dev.to_device(w), dev.to_device(b)
    dy, dpre = dev.zeros(ref.shape), dev.zeros(ref.shape)
    dev.conv2d_fwd_f32(dx_, dw_, db_, dy, B, C, H, W, O, k, k, pad[0], pad[1], stride[0], stride[1], True, dpre, dil=dil)
    assert np.abs(dpre.numpy() - ref).max() <= tol(C * k * k, x, w)
    assert np.abs(dy.numpy() - orc.relu_f32(ref)).max() <= tol(C * k * k, x, w)
    g = rng.standard_normal(ref.shape).astype(np.float32)
    dg = dev.to_device(g)
    gdx, gdw, gdb = dev.zeros(x.shape), dev.zeros(w.shape), dev.zeros(O)
    dev.conv2d_bwd_f32(dg, dx_, dw_, gdx, gdw, gdb, B, C, H, W, O, k, k, pad[0], pad[1], stride[0], stride[1], dil=dil)
    assert dev.check_status() == 0
    rdx, rdw, rdb = orc.conv2d_bwd_f32(g, x, w, pad=pad, stride=stride, dil=dil)
    assert np.abs(gdx.numpy() - rdx).max() <= tol(O * k * k, g, w)
    assert np.abs(gdw.numpy() - rdw).max() <= tol(B * OH * OW, g, x)
    assert np.abs(gdb.numpy() - rdb.ravel()).max() <= tol(B * OH * OW, g, np.ones(1))
    from vtl_b200.capi import VtlbError
    with pytest.raises(VtlbError):
        dev.conv2d_fwd_f32(dx_, dw_, db_, dy, B, C, H, W, O, k, k, pad[0], pad[1], stride[0], stride[1], dil=(0, 1))
