"""The CPU oracle against the reference's own known-answer vectors
(tests/golden/reference_kats.json) and against independent NumPy restatements."""
import json
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def kats():
    with open(os.path.join(HERE, "golden", "reference_kats.json")) as f:
        return json.load(f)


def test_matmul_identity(orc, kats):
    k = kats["matmul_identity"]
    for fn, dt in ((orc.matmul_f32, np.float32), (orc.matmul_f64, np.float64), (orc.matmul_f32_blas, np.float32)):
        assert np.array_equal(fn(np.array(k["a"], dt), np.array(k["b"], dt)), np.array(k["expected"], dt))


def test_linear_forward_backward_f64(orc, kats):
    k = kats["linear_forward_f64"]
    y = orc.linear_fwd_f64(k["x"], k["w"], k["b"])
    assert np.abs(y - np.array(k["expected"])).max() < k["tol"]
    k = kats["linear_backward_f64"]
    dx, dw, db = orc.linear_bwd_f64(k["grad"], k["x"], k["w"])
    assert np.abs(dx - np.array(k["dx"])).max() < k["tol"]
    assert np.abs(dw - np.array(k["dw"])).max() < k["tol"]
    assert np.abs(db - np.array(k["db"])).max() < k["tol"]
    # f32 twin within f32 rounding
    dx32, dw32, db32 = orc.linear_bwd_f32(k["grad"], k["x"], k["w"])
    assert np.abs(dx32 - np.array(k["dx"])).max() < 1e-6
    assert dw32.shape == (2, 3) and db32.shape == (1, 2)


def test_mse_kats(orc, kats):
    c = kats["mse"]["cases"]
    assert orc.mse_f64(c[0]["pred"], c[0]["target"]) < c[0]["tol"]
    assert abs(orc.mse_f64(c[1]["pred"], c[1]["target"]) - c[1]["loss"]) < c[1]["tol"]
    assert abs(float(orc.mse_f32(c[1]["pred"], c[1]["target"])) - c[1]["loss"]) < c[1]["tol"]
    assert abs(orc.mse_bwd_f32(c[2]["pred"], c[2]["target"])[0] - c[2]["grad0"]) < c[2]["tol"]


def test_adam_kats(orc, kats):
    k = kats["adam_one_step_f64"]
    p = k["params"]
    th, m, v = orc.adam_step_f64(k["grad"], k["theta"], k["m"], k["v"], p["b1"], p["b2"], p["lr_t"], p["eps"])
    assert np.abs(th - np.array(k["theta_out"])).max() < 1e-15
    assert np.abs(m - np.array(k["m_out"])).max() < 1e-15
    assert np.abs(v - np.array(k["v_out"])).max() < 1e-15
    th32, m32, v32 = orc.adam_step_f32(k["grad"], k["theta"], k["m"], k["v"], p["b1"], p["b2"], p["lr_t"], p["eps"])
    assert np.abs(th32 - np.array(k["theta_out"])).max() < k["tol"]
    assert np.abs(m32 - np.array(k["m_out"])).max() < k["tol"]
    k = kats["adam_two_steps_f64"]
    th, m, v = np.array(k["theta"]), np.zeros(2), np.zeros(2)
    for _ in range(2):
        th, m, v = orc.adam_step_f64(k["grad"], th, m, v, p["b1"], p["b2"], p["lr_t"], p["eps"])
    assert np.abs(th - np.array(k["theta_out"])).max() < 1e-15


def test_conv2d_kats(orc, kats):
    k = kats["conv2d_4x4"]
    x = np.array(k["input"], np.float32).reshape(1, 1, 4, 4)
    w = np.array(k["weight"], np.float32).reshape(1, 1, 3, 3)
    y = orc.conv2d_fwd_f32(x, w, np.zeros((1, 1), np.float32), pad=k["pad"], stride=k["stride"])
    assert np.abs(y.reshape(4, 4) - np.array(k["forward"])).max() < k["tol_fwd"]
    g = np.array(k["grad_out"], np.float32).reshape(1, 1, 4, 4)
    dx, dw, db = orc.conv2d_bwd_f32(g, x, w, pad=k["pad"], stride=k["stride"])
    assert np.abs(dx.reshape(4, 4) - np.array(k["d_input"])).max() < k["tol_bwd"]
    assert np.abs(dw.reshape(3, 3) - np.array(k["d_weight"])).max() < k["tol_bwd"]
    assert abs(float(db[0, 0]) - k["d_bias"]) < k["tol_bwd"]
    s = kats["conv2d_shape"]
    y = orc.conv2d_fwd_f32(np.zeros(s["in"], np.float32), np.zeros((1, 1, 2, 2), np.float32), None)
    assert list(y.shape) == s["out"]


def test_matmul_c_vs_blas_and_transposes(orc):
    rng = np.random.default_rng(0)
    A = rng.standard_normal((37, 53)).astype(np.float32)
    B = rng.standard_normal((53, 29)).astype(np.float32)
    ref = (A.astype(np.float64) @ B.astype(np.float64)).astype(np.float32)
    for ta, tb, a, b in ((0, 0, A, B), (1, 0, A.T.copy(), B), (0, 1, A, B.T.copy()), (1, 1, A.T.copy(), B.T.copy())):
        got = orc.matmul_f32(a, b, bool(ta), bool(tb))
        # f64 summation order differs between the C loop and dgemm: at most 1 ulp of f32 after rounding
        assert np.abs(got - ref).max() <= 2 * np.spacing(np.abs(ref).max())
        assert np.abs(orc.matmul_f32_blas(a, b, bool(ta), bool(tb)) - ref).max() <= 2 * np.spacing(np.abs(ref).max())


def test_relu_semantics(orc):
    x = np.array([-1.0, -0.0, 0.0, 2.0, np.float32(-1e-45)], np.float32)
    assert np.array_equal(orc.relu_f32(x), np.array([0, -0.0, 0, 2, 0], np.float32))
    g = np.ones(5, np.float32)
    assert np.array_equal(orc.relu_bwd_f32(g, x), np.array([0, 1, 1, 1, 0], np.float32))  # passes at exactly 0


def test_softmax_ce_against_numpy(orc):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((9, 10)).astype(np.float32) * 4
    t = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 9)]
    xs = x.astype(np.float64)
    lse = np.log(np.exp(xs - xs.max(1, keepdims=True)).sum(1)) + xs.max(1)
    ref = np.mean(lse - (t * xs).sum(1))
    assert abs(float(orc.softmax_ce_f32(x, t)) - ref) < 1e-6
    sm = np.exp(xs - xs.max(1, keepdims=True))
    sm /= sm.sum(1, keepdims=True)
    assert np.abs(orc.softmax_ce_bwd_f32(x, t) - (sm - t) / 9).max() < 1e-7


def test_maxpool_standard_semantics(orc):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((2, 3, 6, 8)).astype(np.float32)
    y, idx = orc.maxpool2d_fwd_f32(x)
    ref = x.reshape(2, 3, 3, 2, 4, 2).max(axis=(3, 5))
    assert np.array_equal(y, ref)
    assert np.array_equal(x.ravel()[idx.ravel()], y.ravel())
    g = rng.standard_normal(y.shape).astype(np.float32)
    dx = orc.maxpool2d_bwd_f32(g, idx, x.shape)
    assert np.isclose(dx.sum(), g.sum(), rtol=1e-5) and np.count_nonzero(dx) == g.size


def test_adamw_matches_numpy_f64(orc):
    rng = np.random.default_rng(3)
    g, th, m = (rng.standard_normal(1000).astype(np.float32) for _ in range(3))
    v = rng.random(1000).astype(np.float32)
    b1, b2, lr_t, eps, wd = 0.9, 0.999, 1e-4, 1e-8, 0.01
    m2 = (b1 * m.astype(np.float64) + (1 - b1) * g.astype(np.float64)).astype(np.float32)
    v2 = (b2 * v.astype(np.float64) + (1 - b2) * g.astype(np.float64) * g.astype(np.float64)).astype(np.float32)
    t64 = th.astype(np.float64)
    th2 = (t64 - lr_t * (m2.astype(np.float64) / (np.sqrt(v2.astype(np.float64)) + eps) + wd * t64)).astype(np.float32)
    oth, om, ov = orc.adamw_step_f32(g, th, m, v, b1, b2, lr_t, eps, wd)
    assert np.array_equal(om, m2) and np.array_equal(ov, v2) and np.array_equal(oth, th2)


def test_adamw_kats(orc, kats):
    """One AdamW step against the hand-derived vectors: the oracle's update (textbook operand
    order, the deliberate deviation) and the forensic as-written variant, bit for bit."""
    k = kats["adamw_one_step_f32"]
    p = k["params"]
    args = (k["grad"], k["theta"], k["m"], k["v"], p["b1"], p["b2"], p["lr_t"], p["eps"], p["wd"])
    for name, fn in (("textbook", orc.adamw_step_f32), ("as_written", orc.adamw_step_f32_as_written)):
        th, m, v = fn(*args)
        exp = k[name]
        assert np.array_equal(m, np.array(exp["m_out"], np.float32)), name
        assert np.array_equal(v, np.array(exp["v_out"], np.float32)), name
        want = np.array([np.nan if t is None else t for t in exp["theta_out"]], np.float32)
        assert np.array_equal(th, want, equal_nan=True), name
    # the two differ: the vectors really pin which one is implemented
    assert k["textbook"]["m_out"] != k["as_written"]["m_out"]


def test_adam_lr_t_schedule(orc):
    lr_t, b1t, b2t = orc.adam_lr_t(1e-3, 0.9, 0.999, 0.9, 0.999)
    assert abs(lr_t - 1e-3 * np.sqrt(1 - 0.999) / (1 - 0.9)) < 1e-18
    assert abs(b1t - 0.81) < 1e-15 and abs(b2t - 0.998001) < 1e-15


def test_int8_definition(orc):
    A = np.array([[0.0, 0.0, 0.0, 0.0], [1.0, -2.0, 0.5, 0.25], [127.0, -127.0, 63.5, 0.5]], np.float32)
    q, s = orc.quant_rows_i8(A)
    assert np.array_equal(q[0], [0, 0, 0, 0]) and s[0] == 0
    assert np.array_equal(q[1], [64, -127, 32, 16])  # 63.5 -> 64 and 31.75 -> 32, 15.875 -> 16
    assert np.array_equal(q[2], [127, -127, 64, 0])  # ties to even: 63.5 -> 64, 0.5 -> 0
    assert s[1] == np.float32(2.0) / np.float32(127.0)
    rng = np.random.default_rng(5)
    a = rng.integers(-127, 128, (7, 33), dtype=np.int8)
    w = rng.integers(-127, 128, (5, 33), dtype=np.int8)
    acc = orc.gemm_i8_i32(a, w)
    assert np.array_equal(acc, a.astype(np.int32) @ w.astype(np.int32).T)
    sa, sw = rng.random(7, dtype=np.float32), rng.random(5, dtype=np.float32)
    b = rng.standard_normal(5).astype(np.float32)
    y = orc.dequant_bias_relu(acc, sa, sw, b, True)
    ref = np.maximum(acc.astype(np.float32) * (sa[:, None] * sw[None, :]) + b[None, :], 0).astype(np.float32)
    assert np.array_equal(y, ref)


def test_mlp_oracle_step_decreases_loss(orc):
    rng = np.random.default_rng(1)
    W1 = (rng.uniform(-1, 1, (16, 8)) * np.sqrt(6 / 8)).astype(np.float32)
    W2 = (rng.uniform(-1, 1, (4, 16)) * np.sqrt(6 / 16)).astype(np.float32)
    net = orc.MLPOracle([W1, W2], [np.zeros(16), np.zeros(4)], [True, False], lr=1e-2)
    X = rng.random((32, 8), dtype=np.float32)
    T = np.eye(4, dtype=np.float32)[rng.integers(0, 4, 32)]
    losses = [float(net.step(X, T)) for _ in range(30)]
    assert losses[-1] < losses[0]
    blas = orc.MLPOracle([W1, W2], [np.zeros(16), np.zeros(4)], [True, False], lr=1e-2, blas=True)
    assert abs(float(blas.step(X, T)) - losses[0]) < 1e-6


def test_oracle_thread_count_can_be_raised_after_load():
    """The benchmark's CPU arm sets the OpenMP thread count itself (a launcher may have exported
    OMP_NUM_THREADS=1 before the library was loaded)."""
    from oracle import oracle
    oracle.build()
    before = oracle.max_threads()
    try:
        oracle.set_threads(2)
        assert oracle.max_threads() == 2
        oracle.set_threads(1)
        assert oracle.max_threads() == 1
    finally:
        oracle.set_threads(before)
    assert oracle.max_threads() == before


def test_initialiser_restatement(orc):
    """compute_fans keeps the reference's product over shape[1..] (nn/internal/init.v:21-33); the
    counter-based fills have the moments variance_scaled asks for."""
    assert orc.compute_fans([256, 784]) == (256 * 784, 784 * 784)
    assert orc.compute_fans([64, 32, 3, 3]) == (64 * 32 * 9, 32 * 32 * 9)
    std = orc.variance_scaled_std([64, 32, 3, 3], 2.0, "fan_in")
    assert abs(std - np.sqrt(2.0 / (64 * 288))) < 1e-15
    assert abs(orc.variance_scaled_std([4, 6], 2.0, "fan_avg") - np.sqrt(4.0 / (24 + 36))) < 1e-15
    n = 200000
    u = orc.init_uniform_f32(n, -1.0, 1.0, 3)
    assert u.dtype == np.float32 and u.min() >= -1.0 and u.max() < 1.0
    assert abs(u.mean()) < 0.01 and abs(u.std() - 1 / np.sqrt(3)) < 0.01
    g = orc.init_normal_f32(n, 0.0, 2.0, 4)
    assert abs(g.mean()) < 0.02 and abs(g.std() - 2.0) < 0.02
    assert np.array_equal(orc.init_normal_f32(10, 0.0, 2.0, 4), g[:10])  # element i depends on (seed, i) only


def test_reference_optimizer_tests_hold_for_the_oracle(orc):
    """The assertions of the reference's own optimizer tests, on the oracle: SGD 5.0 - 0.1 * 1.0 = 4.9
    (nn/optimizers/optimizer_test.v:16-27) and the Adam f32 / f64 steps from zero moments moving theta
    down and the first moment up (optimizer_test.v:39-67: grad [1, 2], theta [5, 5], beta 0.9 / 0.999,
    lr_t 0.001, eps 1e-8)."""
    theta = orc.sgd_step_f32(np.array([1.0], np.float32), np.array([5.0], np.float32), 0.1)
    assert abs(float(theta[0]) - 4.9) < 1e-6
    g = [1.0, 2.0]
    for step, dt in ((orc.adam_step_f32, np.float32), (orc.adam_step_f64, np.float64)):
        th, m, v = step(np.array(g, dt), np.array([5.0, 5.0], dt), np.zeros(2, dt), np.zeros(2, dt),
                        0.9, 0.999, 0.001, 1e-8)
        assert th[0] < 5.0 and th[1] < 5.0 and m[0] > 0.0
        # first step from zero moments: m = 0.1 g, v = 0.001 g^2, so theta moves by lr_t * 0.1 / sqrt(0.001)
        want = 5.0 - 0.001 * (0.1 * np.array(g)) / (np.sqrt(0.001 * np.array(g) ** 2) + 1e-8)
        assert np.allclose(th, want, rtol=0, atol=2e-6 if dt == np.float32 else 1e-12)


def test_inputs_of_the_reference_device_comparison_tests(orc):
    """The reference compares its GPU paths with its CPU functions on a few fixed inputs.  The inputs
    are simple enough for the CPU side to be worked out by hand, which pins the oracle:
    ReLU of [[2, -1], [0.5, -3]] (nn/layers/activation_vulkan_relu_f32_d_vulkan_test.v:12-14);
    all-ones 1x2x8x8 input and 4x2x3x3 weights, zero bias, padding 1 and 0
    (nn/internal/conv2d_vulkan_forward_f32_d_vulkan_test.v:19-23, conv2d_vulkan_backward_f32_d_vulkan_test.v:12-34):
    an output is 2 x (taps inside the image), a weight gradient under all-ones upstream is the number
    of output positions whose tap falls inside the image."""
    assert np.array_equal(orc.relu_f32(np.array([[2, -1], [0.5, -3]], np.float32)),
                          np.array([[2, 0], [0.5, 0]], np.float32))
    x, w, b = np.ones((1, 2, 8, 8), np.float32), np.ones((4, 2, 3, 3), np.float32), np.zeros((1, 4), np.float32)
    y = orc.conv2d_fwd_f32(x, w, b, pad=(1, 1), stride=(1, 1))
    assert y.shape == (1, 4, 8, 8)
    inside = np.array([2] + [3] * 6 + [2])  # taps of a 3-wide window that fall inside an 8-long axis
    assert np.array_equal(y[0, 0], 2.0 * np.outer(inside, inside)) and (y == y[:, :1]).all()
    y0 = orc.conv2d_fwd_f32(x, w, b, pad=(0, 0), stride=(1, 1))
    assert y0.shape == (1, 4, 6, 6) and (y0 == 18.0).all()
    for pad, out in ((0, 6), (1, 8)):
        g = np.ones((1, 4, out, out), np.float32)
        dx, dw, db = orc.conv2d_bwd_f32(g, x, w, pad=(pad, pad), stride=(1, 1))
        # tap (a, b) meets the image at out - |a - 1| * pad positions per axis
        per_axis = np.array([out - pad, out, out - pad]) if pad else np.array([out] * 3)
        assert np.array_equal(dw[0, 0], np.outer(per_axis, per_axis).astype(np.float32)) and (dw == dw[:1, :1]).all()
        assert (db.ravel() == out * out).all()
        # every input pixel feeds 4 channels x (windows that cover it)
        cover = np.array([1, 2] + [3] * 4 + [2, 1]) if pad == 0 else inside
        assert np.array_equal(dx[0, 0], 4.0 * np.outer(cover, cover)) and (dx == dx[:, :1]).all()
