"""ReLU, losses and Adam/AdamW kernels against the oracle."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [1, 7, 1024, 100003])
def test_relu_fwd_bwd_bit_exact(dev, orc, n):
    rng = np.random.default_rng(n)
    x = rng.standard_normal(n).astype(np.float32)
    x[::5] = 0.0
    if n > 3:
        x[3] = -0.0
    g = rng.standard_normal(n).astype(np.float32)
    dx, dg = dev.to_device(x), dev.to_device(g)
    dy, dd = dev.empty(n), dev.empty(n)
    dev.relu_fwd_f32(dx, dy, n)
    dev.relu_bwd_f32(dg, dx, dd, n)
    assert np.array_equal(dy.numpy().view(np.uint32), orc.relu_f32(x).view(np.uint32))
    assert np.array_equal(dd.numpy().view(np.uint32), orc.relu_bwd_f32(g, x).view(np.uint32))


def test_mse_reference_kats(dev):
    """nn/loss/loss_test.v:20-51: identical -> 0; [2,2] vs [0,0] -> 4.0; grad of [3,1] vs [1,1] -> 2.0."""
    def run(p, t):
        p, t = np.asarray(p, np.float32), np.asarray(t, np.float32)
        dp, dt = dev.to_device(p), dev.to_device(t)
        dl, dg = dev.zeros(1), dev.zeros(p.size)
        dev.mse_fwd_bwd_f32(dp, dt, p.size, p.size, dl, dg)
        return float(dl.numpy()[0]), dg.numpy()
    assert run([1, 2, 3, 4], [1, 2, 3, 4])[0] == 0.0
    assert abs(run([2, 2], [0, 0])[0] - 4.0) < 1e-6
    assert abs(run([3, 1], [1, 1])[1][0] - 2.0) < 1e-6


@pytest.mark.parametrize("n", [10, 640, 64 * 4096])
def test_mse_vs_oracle(dev, orc, n):
    rng = np.random.default_rng(n)
    p = rng.standard_normal(n).astype(np.float32)
    t = rng.standard_normal(n).astype(np.float32)
    dp, dt = dev.to_device(p), dev.to_device(t)
    dl, dg = dev.zeros(1), dev.zeros(n)
    dev.mse_fwd_bwd_f32(dp, dt, n, n, dl, dg)
    assert np.array_equal(dg.numpy().view(np.uint32), orc.mse_bwd_f32(p, t).view(np.uint32))
    # the oracle sums sequentially in f32 (as the reference does); its own rounding
    # noise grows with n, the kernel sums in f64: compare at 1e-4 relative
    assert abs(float(dl.numpy()[0]) - float(orc.mse_f32(p, t))) <= 1e-4 * float(orc.mse_f64(p, t))
    assert abs(float(dl.numpy()[0]) - orc.mse_f64(p, t)) <= 1e-6 * orc.mse_f64(p, t)


@pytest.mark.parametrize("B,C", [(1, 2), (256, 10), (1000, 37)])
def test_softmax_ce_vs_oracle(dev, orc, B, C):
    rng = np.random.default_rng(B * C)
    x = (rng.standard_normal((B, C)) * 3).astype(np.float32)
    t = np.eye(C, dtype=np.float32)[rng.integers(0, C, B)]
    dx, dt = dev.to_device(x), dev.to_device(t)
    dl, dg = dev.zeros(1), dev.zeros((B, C))
    dev.softmax_ce_fwd_bwd_f32(dx, dt, B, C, B, dl, dg)
    assert abs(float(dl.numpy()[0]) - float(orc.softmax_ce_f32(x, t))) <= 1e-6 * max(1.0, abs(float(orc.softmax_ce_f32(x, t))))
    ref = orc.softmax_ce_bwd_f32(x, t)
    assert np.abs(dg.numpy() - ref).max() <= 1e-7


def _adam_inputs(rng, n):
    g = rng.standard_normal(n).astype(np.float32)
    th = rng.standard_normal(n).astype(np.float32)
    m = (rng.standard_normal(n) * 0.1).astype(np.float32)
    v = (rng.random(n) * 0.01).astype(np.float32)
    return g, th, m, v


@pytest.mark.parametrize("sizes", [[3], [1, 5, 4096, 4097], [200704, 256, 2560, 10], [7] * 130])
@pytest.mark.parametrize("kind", ["adam", "adamw"])
def test_adam_multi_tensor_bit_exact(dev, orc, sizes, kind):
    rng = np.random.default_rng(len(sizes) + sizes[0])
    host, bufs, table = [], [], []
    for n in sizes:
        arrs = _adam_inputs(rng, n)
        host.append(arrs)
        d = [dev.to_device(a) for a in arrs]
        bufs.append(d)
        table.append((d[0], d[1], d[2], d[3], n))
    tb = dev.adam_table(table)
    b1, b2, lr_t, eps, wd = 0.9, 0.999, 0.0031, 1e-8, 0.01
    for step in range(2):
        if kind == "adam":
            dev.adam_step_f32(tb, b1, b2, lr_t, eps, zero_grad=(step == 1))
        else:
            dev.adamw_step_f32(tb, b1, b2, lr_t, eps, wd, zero_grad=(step == 1))
    for (g, th, m, v), d in zip(host, bufs):
        for step in range(2):
            if kind == "adam":
                th, m, v = orc.adam_step_f32(g, th, m, v, b1, b2, lr_t, eps)
            else:
                th, m, v = orc.adamw_step_f32(g, th, m, v, b1, b2, lr_t, eps, wd)
        for got, ref, name in ((d[1], th, "theta"), (d[2], m, "m"), (d[3], v, "v")):
            assert np.array_equal(got.numpy().view(np.uint32), ref.view(np.uint32)), name
        assert not d[0].numpy().any(), "gradients must be cleared by zero_grad"


def test_adam_reference_kat(dev):
    """nn/optimizers/adam_cuda_d_cuda_test.v:8-34 inputs; expected values from the
    formula of adam_step_f64.v evaluated in Python floats (f32 kernel: 1e-6)."""
    g = np.array([1.0, 2.0, 0.5]); th = np.array([3.0, 4.0, 5.0])
    m = np.array([0.1, 0.2, 0.3]); v = np.array([0.01, 0.02, 0.03])
    m2 = 0.9 * m + (1 - 0.9) * g
    v2 = 0.999 * v + (1 - 0.999) * g * g
    th2 = th - 0.01 * m2 / (np.sqrt(v2) + 1e-8)
    d = [dev.to_device(a.astype(np.float32)) for a in (g, th, m, v)]
    dev.adam_step_f32(dev.adam_table([(d[0], d[1], d[2], d[3], 3)]), 0.9, 0.999, 0.01, 1e-8, False)
    assert np.abs(d[1].numpy() - th2).max() < 1e-6
    assert np.abs(d[2].numpy() - m2).max() < 1e-6
    assert np.abs(d[3].numpy() - v2).max() < 1e-6


def test_adamw_hand_derived_kat(dev):
    """One AdamW step on the hand-derived vector of tests/golden (nn/optimizers/adamw.v:78-106
    with the moments in the textbook operand order): theta, m and v bit for bit, and NOT the
    values the update would give with the closures' operands as written."""
    import json
    import os
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_kats.json")) as f:
        k = json.load(f)["adamw_one_step_f32"]
    p = k["params"]
    d = [dev.to_device(np.array(k[n], np.float32)) for n in ("grad", "theta", "m", "v")]
    dev.adamw_step_f32(dev.adam_table([(d[0], d[1], d[2], d[3], len(k["grad"]))]), p["b1"], p["b2"], p["lr_t"],
                       p["eps"], p["wd"], False)
    exp = k["textbook"]
    for got, name in ((d[1], "theta_out"), (d[2], "m_out"), (d[3], "v_out")):
        assert np.array_equal(got.numpy().view(np.uint32), np.array(exp[name], np.float32).view(np.uint32)), name
    assert not np.array_equal(d[2].numpy(), np.array(k["as_written"]["m_out"], np.float32))
