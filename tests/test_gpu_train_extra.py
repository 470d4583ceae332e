"""Training steps through the host mirror with the layers and optimizers that sit next to the GEMM
layers in the reference's examples (BatchNorm1D, softmax, average pooling; SGD, RMSProp), against
a step composed from the CPU oracle's functions on identical seeded inputs."""
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


def close(a, b, tol):
    return float(np.abs(np.asarray(a, np.float64) - np.asarray(b, np.float64)).max()) <= tol


@pytest.mark.parametrize("optimizer", ["sgd", "rmsprop"])
def test_mlp_with_batchnorm_and_softmax(sess, orc, optimizer):
    from vtl_b200 import host
    rng = np.random.default_rng(21)
    B = 32
    X = rng.standard_normal((B, 6)).astype(np.float32)
    T = np.eye(4, dtype=np.float32)[rng.integers(0, 4, B)]
    W1, b1 = (rng.standard_normal((8, 6)) * 0.5).astype(np.float32), (rng.standard_normal(8) * 0.1).astype(np.float32)
    W2, b2 = (rng.standard_normal((4, 8)) * 0.5).astype(np.float32), (rng.standard_normal(4) * 0.1).astype(np.float32)
    gamma, beta = np.ones(8, np.float32), np.zeros(8, np.float32)
    rm, rv = np.zeros(8, np.float32), np.ones(8, np.float32)

    m = host.Model(sess)
    m.input([6]); m.linear(8); m.batchnorm1d(8); m.relu(); m.linear(4); m.softmax()
    m.mse_loss()
    if optimizer == "sgd":
        m.sgd(lr=0.1)
    else:
        m.rmsprop(lr=0.01, alpha=0.9, eps=1e-8, weight_decay=0.001)
    assert m.num_params() == 6  # W1, b1, gamma, beta, W2, b2
    for i, p in enumerate((W1, b1, gamma, beta, W2, b2)):
        m.set_param(i, p)
    dX, dT = sess.dev.to_device(X), sess.dev.to_device(T)
    params = [W1, b1, gamma, beta, W2, b2]
    sq = [np.zeros_like(p) for p in params]
    for step in range(4):
        loss = m.train_step(dX, X.shape, dT, T.shape)
        # the same step from the oracle's pieces
        W1, b1, gamma, beta, W2, b2 = params
        h1 = orc.linear_fwd_f32(X, W1, b1)
        y, mean, var, rm, rv = orc.batchnorm1d_train_f32(h1, gamma, beta, 1e-5, rm, rv, 0.1)
        r = orc.relu_f32(y)
        z = orc.linear_fwd_f32(r, W2, b2)
        p = orc.softmax_fwd_f32(z)
        ref_loss = orc.mse_f32(p, T)
        dz = orc.softmax_bwd_f32(orc.mse_bwd_f32(p, T), z)
        dr, dW2, db2 = orc.linear_bwd_f32(dz, r, W2)
        dy = orc.relu_bwd_f32(dr, y)
        dh1, _, _ = orc.batchnorm1d_bwd_f32(dy, h1, gamma, mean, var, 1e-5)
        _, dW1, db1 = orc.linear_bwd_f32(dh1, X, W1)
        # gamma and beta get no gradient: the reference registers the gate with the input as its only parent
        grads = [dW1, db1.reshape(-1), np.zeros(8, np.float32), np.zeros(8, np.float32), dW2, db2.reshape(-1)]
        for i in range(6):
            if optimizer == "sgd":
                params[i] = orc.sgd_step_f32(grads[i], params[i], 0.1)
            else:
                params[i], sq[i] = orc.rmsprop_step_f32(grads[i], params[i], sq[i], 0.01, 0.9, 1e-8, 0.001)
        assert abs(loss - float(ref_loss)) <= 1e-5 * max(1.0, abs(float(ref_loss))), (step, loss, ref_loss)
        # RMSProp divides by sqrt(sq) ~ |g|: its steps are +-lr whatever the size of g, so compare loosely
        tol = 2e-4 if optimizer == "sgd" else 2e-3
        for i in range(6):
            if optimizer == "rmsprop" and i == 1:
                # b1 feeds a BatchNorm, which removes the batch mean: its gradient is rounding noise
                # (~1e-8), and RMSProp turns noise into steps of +-lr/sqrt(1-alpha) in either
                # direction.  Nothing to compare; the SGD run covers this parameter.
                continue
            assert close(m.get_param(i), params[i].reshape(-1), tol), (step, i)
        if optimizer == "rmsprop":
            params[1] = m.get_param(1).copy()  # keep both sides on the same b1 (it does not change h1 - mean)
            for i in (0, 4):
                assert close(m.get_sq_avg(i), sq[i].reshape(-1), 1e-4 * max(1.0, float(np.abs(sq[i]).max())))
    assert close(m.running_stat(0, 8), rm, 1e-4) and close(m.running_stat(0, 8, variance=True), rv, 1e-4)
    assert np.array_equal(m.get_param(2), np.ones(8, np.float32) if optimizer == "sgd" else m.get_param(2))
    m.close(); dX.free(); dT.free()


def test_cnn_with_average_pools(sess, orc):
    from vtl_b200 import host
    rng = np.random.default_rng(22)
    B = 8
    X = rng.standard_normal((B, 2, 6, 6)).astype(np.float32)
    T = rng.standard_normal((B, 2)).astype(np.float32)
    Wc, bc = (rng.standard_normal((3, 2, 3, 3)) * 0.3).astype(np.float32), (rng.standard_normal(3) * 0.1).astype(np.float32)
    Wl, bl = (rng.standard_normal((2, 3)) * 0.5).astype(np.float32), np.zeros(2, np.float32)
    m = host.Model(sess)
    m.input([2, 6, 6]); m.conv2d(2, 3, (3, 3), padding=(1, 1)); m.relu(); m.avgpool2d((2, 2), (0, 0), (2, 2))
    m.global_avgpool2d(); m.flatten(); m.linear(2)
    m.mse_loss(); m.sgd(lr=0.05)
    for i, p in enumerate((Wc, bc, Wl, bl)):
        m.set_param(i, p)
    dX, dT = sess.dev.to_device(X), sess.dev.to_device(T)
    params = [Wc, bc, Wl, bl]
    for step in range(3):
        loss = m.train_step(dX, X.shape, dT, T.shape)
        Wc, bc, Wl, bl = params
        c = orc.conv2d_fwd_f32(X, Wc, bc, pad=(1, 1))
        r = orc.relu_f32(c)
        a = orc.avgpool2d_fwd_f32(r, (2, 2), (0, 0), (2, 2))
        gp = orc.global_avgpool2d_fwd_f32(a)
        f = gp.reshape(B, 3)
        out = orc.linear_fwd_f32(f, Wl, bl)
        ref_loss = orc.mse_f32(out, T)
        df, dWl, dbl = orc.linear_bwd_f32(orc.mse_bwd_f32(out, T), f, Wl)
        da = orc.global_avgpool2d_bwd_f32(df.reshape(B, 3, 1, 1), a.shape)
        dr = orc.avgpool2d_bwd_f32(da, r.shape, (2, 2), (0, 0), (2, 2))
        dc = orc.relu_bwd_f32(dr, c)
        _, dWc, dbc = orc.conv2d_bwd_f32(dc, X, Wc, pad=(1, 1))
        grads = [dWc, dbc.reshape(-1), dWl, dbl.reshape(-1)]
        params = [orc.sgd_step_f32(g, p, 0.05) for g, p in zip(grads, params)]
        assert abs(loss - float(ref_loss)) <= 1e-5 * max(1.0, abs(float(ref_loss)))
        for i in range(4):
            assert close(m.get_param(i), params[i].reshape(-1), 2e-4), (step, i)
    m.close(); dX.free(); dT.free()


def test_inference_path_uses_running_statistics(sess, orc):
    """BatchNorm1D on an input that does not require a gradient normalises with the running
    statistics (nn/layers/batchnorm.v:70-75); Model.forward feeds such an input."""
    from vtl_b200 import host
    rng = np.random.default_rng(23)
    X = rng.standard_normal((5, 4)).astype(np.float32)
    m = host.Model(sess)
    m.input([4]); m.batchnorm1d(4); m.softmax()
    gamma, beta = rng.uniform(0.5, 1.5, 4).astype(np.float32), rng.standard_normal(4).astype(np.float32)
    m.set_param(0, gamma); m.set_param(1, beta)
    dX, dY = sess.dev.to_device(X), sess.dev.zeros((5, 4))
    m.forward(dX, X.shape, dY)
    bn = orc.batchnorm1d_infer_f32(X, gamma, beta, np.zeros(4, np.float32), np.ones(4, np.float32), 1e-5)
    want = orc.softmax_fwd_f32(bn)
    assert close(dY.numpy(), want, 1e-6)
    m.close(); dX.free(); dY.free()
