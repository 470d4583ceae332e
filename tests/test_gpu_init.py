"""Parameter initialisers (nn/internal/init.v:21-70): compute_fans as written, variance_scaled,
kaiming_uniform / kaiming_normal, and the layers' default Kaiming-normal weights
(nn/layers/linear.v:25, nn/layers/conv2d.v:49) against the NumPy restatement."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def sess():
    from vtl_b200 import capi, host
    if capi.device_count() == 0:
        pytest.skip("no CUDA device")
    s = host.Session(0)
    yield s
    s.dev.sync()
    assert s.dev.check_status() == 0
    s.close()


@pytest.mark.parametrize("n,lo,hi,seed", [(1, -1.0, 1.0, 0), (1000, -0.5, 0.25, 7), (100003, 0.0, 3.0, 2 ** 63 + 5)])
def test_uniform_fill_bit_exact(dev, orc, n, lo, hi, seed):
    d = dev.empty(n)
    dev.init_uniform_f32(d, n, lo, hi, seed)
    got, ref = d.numpy(), orc.init_uniform_f32(n, lo, hi, seed)
    assert np.array_equal(got.view(np.uint32), ref.view(np.uint32))
    assert got.min() >= lo and got.max() <= hi


@pytest.mark.parametrize("n,mu,sigma,seed", [(3, 0.0, 1.0, 1), (65537, 0.5, 0.02, 99)])
def test_normal_fill_matches_restatement(dev, orc, n, mu, sigma, seed):
    d = dev.empty(n)
    dev.init_normal_f32(d, n, mu, sigma, seed)
    got, ref = d.numpy(), orc.init_normal_f32(n, mu, sigma, seed)
    # Box-Muller runs in f64 on both sides; log and cos may differ in the last f64 bit between the
    # two math libraries, which can move the f32 rounding of a value by one ulp
    ulp = np.spacing(np.abs(ref).astype(np.float32))
    assert np.all(np.abs(got - ref) <= ulp)
    assert np.mean(got == ref) > 0.999


def test_compute_fans_keeps_the_reference_arithmetic(orc):
    from vtl_b200 import host
    for shape in ([256, 784], [10, 256], [32, 3, 3, 3], [64, 32, 3, 3], [5, 7, 1, 1]):
        assert host.compute_fans(shape) == orc.compute_fans(shape)
    assert host.compute_fans([256, 784]) == (256 * 784, 784 * 784)          # not (784, 256)
    assert host.compute_fans([64, 32, 3, 3]) == (64 * 288, 32 * 288)
    from vtl_b200 import capi
    with pytest.raises(capi.VtlbError):
        host.compute_fans([5])


@pytest.mark.parametrize("shape", [[512, 1024], [64, 32, 3, 3]])
def test_variance_scaled_moments_and_limits(sess, orc, shape):
    from vtl_b200 import host
    n = int(np.prod(shape))
    for mode, name in ((host.FAN_IN, "fan_in"), (host.FAN_OUT, "fan_out"), (host.FAN_AVG, "fan_avg")):
        std = orc.variance_scaled_std(shape, 2.0, name)
        u = sess.variance_scaled(shape, 2.0, mode, host.UNIFORM, seed=11)
        limit = np.float32(np.sqrt(3.0) * std)
        assert np.array_equal(u.ravel(), orc.init_uniform_f32(n, -limit, limit, 11))
        assert abs(u.std() - std) < 0.02 * std and abs(u.mean()) < 4 * std / np.sqrt(n)
        g = sess.variance_scaled(shape, 2.0, mode, host.NORMAL, seed=12)
        assert abs(g.std() - std) < 0.02 * std and abs(g.mean()) < 4 * std / np.sqrt(n)
        assert abs(np.mean(np.abs(g) < std) - 0.6827) < 0.01   # a normal, not just the right variance
    k = sess.kaiming_normal(shape, seed=5)
    assert np.array_equal(k, sess.variance_scaled(shape, 2.0, host.FAN_IN, host.NORMAL, 5))
    assert not np.array_equal(k, sess.kaiming_normal(shape, seed=6))


def test_layers_start_from_seeded_kaiming_normal(sess, orc):
    """A model built through the API alone has trainable (non-zero) weights, zero biases, the std of
    kaiming_normal on the reference's fans, and the same weights again for the same seed."""
    from vtl_b200 import host

    def build():
        sess.set_seed(1234)
        m = host.Model(sess)
        m.input([3, 8, 8])
        m.conv2d(3, 16, (3, 3), padding=(1, 1)); m.relu()
        m.flatten()
        m.linear(32)
        m.mse_loss()
        m.adam(lr=1e-3)
        return m

    m = build()
    w_conv, b_conv, w_lin, b_lin = (m.get_param(i) for i in range(4))
    assert not b_conv.any() and not b_lin.any()
    for w, shape in ((w_conv, [16, 3, 3, 3]), (w_lin, [32, 16 * 8 * 8])):
        std = orc.variance_scaled_std(shape, 2.0, "fan_in")
        assert abs(w.std() - std) < 0.1 * std
    m2 = build()
    assert np.array_equal(m2.get_param(0), w_conv) and np.array_equal(m2.get_param(2), w_lin)
    assert not np.array_equal(w_conv[:100], w_lin[:100])  # layers draw from different streams
    # and it trains: the loss falls over a few steps on a fixed batch
    rng = np.random.default_rng(0)
    X = rng.standard_normal((16, 3, 8, 8)).astype(np.float32)
    T = rng.standard_normal((16, 32)).astype(np.float32)
    dX, dT = sess.dev.to_device(X), sess.dev.to_device(T)
    losses = [m.train_step(dX, X.shape, dT, T.shape) for _ in range(10)]
    assert losses[-1] < losses[0]
    m.close(); m2.close()
