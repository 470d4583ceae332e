"""Whole training steps through the C++ host mirror of vtl's Sequential / autograd /
optimizer API, against the step-by-step CPU oracle on identical seeded inputs."""
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


@pytest.fixture(params=["tensor_cores_only", "small_products_on_cuda_cores"], autouse=True)
def session_gemm_path(request, sess):
    """Every training test runs with all f32 products on tcgen05 and with the default routing."""
    sess.dev.set_small_gemm_limit(0.0 if request.param == "tensor_cores_only" else 1.4e8)
    yield
    sess.dev.set_small_gemm_limit(1.4e8)


def kaiming_uniform(rng, out_f, in_f):
    return (rng.uniform(-1, 1, (out_f, in_f)) * np.sqrt(6.0 / in_f)).astype(np.float32)


def build_mlp(sess, dims, relu_after, opt="adam", **kw):
    from vtl_b200 import host
    m = host.Model(sess)
    m.input([dims[0]])
    for i, d in enumerate(dims[1:]):
        m.linear(d)
        if relu_after[i]:
            m.relu()
    m.mse_loss()
    (m.adam if opt == "adam" else m.adamw)(**kw)
    return m


def bound(K, a, b):
    return 1e-5 * np.sqrt(K) * float(np.abs(a).max()) * float(np.abs(b).max())


@pytest.mark.parametrize("fuse", [True, False])
def test_mlp_config1_gradients_and_steps(sess, orc, fuse):
    """Baseline config 1: 784 -> 256 -> 10, batch 64, MSE vs one-hot, Adam lr 1e-3."""
    rng = np.random.default_rng(1)
    X = rng.random((64, 784), dtype=np.float32)
    T = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 64)]
    W1, W2 = kaiming_uniform(rng, 256, 784), kaiming_uniform(rng, 10, 256)
    b1, b2 = np.zeros(256, np.float32), np.zeros(10, np.float32)
    m = build_mlp(sess, [784, 256, 10], [True, False], lr=1e-3)
    m.set_fuse_relu(fuse)
    for i, p in enumerate((W1, b1, W2, b2)):
        m.set_param(i, p)
    ref = orc.MLPOracle([W1, W2], [b1, b2], [True, False], lr=1e-3)
    dX, dT = sess.dev.to_device(X), sess.dev.to_device(T)

    # gradients of the first step (no update)
    loss = m.train_step(dX, X.shape, dT, T.shape, update=False)
    rloss, y, dWs, dbs, dIn = ref.grads(X, T)
    assert abs(loss - float(rloss)) <= 1e-5 * max(1.0, abs(float(rloss)))
    h = orc.relu_f32(orc.linear_fwd_f32(X, W1, b1))
    g2 = y - T
    assert np.abs(m.get_grad(2).reshape(10, 256) - dWs[1]).max() <= bound(64, g2, h) + 1e-6
    assert np.abs(m.get_grad(3) - dbs[1].ravel()).max() <= bound(64, g2, np.ones(1)) + 1e-6
    assert np.abs(m.get_grad(0).reshape(256, 784) - dWs[0]).max() <= bound(64, g2, X) * 4 + 1e-6
    assert np.abs(m.get_grad(1) - dbs[0].ravel()).max() <= bound(64, g2, np.ones(1)) * 4 + 1e-6
    assert np.abs(m.input_grad(X.shape) - dIn).max() <= bound(256, g2, W1) * 4 + 1e-6

    m.zero_grad()  # a second backprop would otherwise accumulate onto these gradients

    # 20 full steps.  Adam divides by sqrt(v): where a gradient is close to zero, a last-bit
    # difference between the f64-accumulated oracle GEMM and the GPU GEMM moves a weight by
    # up to lr in one step, so trajectories drift apart slowly; the bounds below allow that.
    gl, rl = [], []
    for _ in range(20):
        gl.append(m.train_step(dX, X.shape, dT, T.shape))
        rl.append(float(ref.step(X, T)))
    assert np.allclose(gl[:3], rl[:3], rtol=5e-5, atol=1e-6), (gl[:3], rl[:3])
    assert np.allclose(gl, rl, rtol=2e-3, atol=1e-6), (gl[-3:], rl[-3:])
    assert rl[-1] < rl[0]
    for i, r in enumerate((ref.W[0], ref.b[0], ref.W[1], ref.b[1])):
        diff = np.abs(m.get_param(i) - r.ravel())
        assert diff.max() <= 5e-3 and np.quantile(diff, 0.99) <= 5e-4 and np.median(diff) <= 2e-5, (i, diff.max())
    m.close()


def test_adamw_deep_mlp_small(sess, orc):
    """Config 4 in miniature: 4 Linear layers of width 128 with ReLU between, MSE vs N(0,1)
    targets, AdamW lr 1e-4 wd 0.01."""
    rng = np.random.default_rng(4)
    dims = [128] * 5
    relu_after = [True, True, True, False]
    X = rng.standard_normal((256, 128)).astype(np.float32)
    T = rng.standard_normal((256, 128)).astype(np.float32)
    Ws = [kaiming_uniform(rng, 128, 128) for _ in range(4)]
    bs = [np.zeros(128, np.float32) for _ in range(4)]
    m = build_mlp(sess, dims, relu_after, opt="adamw", lr=1e-4, weight_decay=0.01)
    for i in range(4):
        m.set_param(2 * i, Ws[i])
        m.set_param(2 * i + 1, bs[i])
    ref = orc.MLPOracle(Ws, bs, relu_after, lr=1e-4, weight_decay=0.01)
    dX, dT = sess.dev.to_device(X), sess.dev.to_device(T)
    for _ in range(5):
        gl, rl = m.train_step(dX, X.shape, dT, T.shape), float(ref.step(X, T))
        assert abs(gl - rl) <= 1e-4 * abs(rl)
    for i in range(4):
        assert np.abs(m.get_param(2 * i) - ref.W[i].ravel()).max() <= 5e-5
        assert np.abs(m.get_moment(2 * i, second=False) - ref.mW[i].ravel()).max() <= 1e-3 * np.abs(ref.mW[i]).max() + 1e-7
    m.close()


def test_cnn_config3_small_batch(sess, orc):
    """Config 3 topology at batch 4: conv3x3 3->32 +ReLU, conv3x3 32->64 +ReLU, 2x2 max-pool,
    Linear 16384->10, softmax cross-entropy, Adam lr 1e-3."""
    from vtl_b200 import host
    rng = np.random.default_rng(3)
    B = 4
    X = rng.standard_normal((B, 3, 32, 32)).astype(np.float32)
    T = np.eye(10, dtype=np.float32)[rng.integers(0, 10, B)]
    w1 = (rng.uniform(-1, 1, (32, 3, 3, 3)) * np.sqrt(6.0 / 27)).astype(np.float32)
    w2 = (rng.uniform(-1, 1, (64, 32, 3, 3)) * np.sqrt(6.0 / 288)).astype(np.float32)
    w3 = kaiming_uniform(rng, 10, 16384)
    z = lambda n: np.zeros(n, np.float32)
    m = host.Model(sess)
    m.input([3, 32, 32])
    m.conv2d(3, 32, (3, 3), padding=(1, 1)); m.relu()
    m.conv2d(32, 64, (3, 3), padding=(1, 1)); m.relu()
    m.maxpool2d((2, 2), (0, 0), (2, 2))
    m.flatten()
    m.linear(10)
    m.softmax_cross_entropy_loss()
    m.adam(lr=1e-3)
    for i, p in enumerate((w1, z(32), w2, z(64), w3, z(10))):
        m.set_param(i, p)
    ref = orc.SequentialOracle([("conv2d", w1, z(32), (1, 1), (1, 1)), ("relu",),
                                ("conv2d", w2, z(64), (1, 1), (1, 1)), ("relu",),
                                ("maxpool2d", (2, 2), (0, 0), (2, 2)), ("flatten",),
                                ("linear", w3, z(10))], loss="sce", lr=1e-3)
    dX, dT = sess.dev.to_device(X), sess.dev.to_device(T)
    loss = m.train_step(dX, X.shape, dT, T.shape, update=False)
    rloss, _, rg, rdx = ref.grads(X, T)
    assert abs(loss - float(rloss)) <= 1e-5 * abs(float(rloss))
    for i in range(6):
        g = m.get_grad(i)
        scale = max(float(np.abs(rg[i]).max()), 1e-6)
        assert np.abs(g - rg[i].ravel()).max() <= 2e-4 * scale, (i, np.abs(g - rg[i].ravel()).max(), scale)
    assert np.abs(m.input_grad(X.shape) - rdx).max() <= 2e-4 * float(np.abs(rdx).max())
    m.zero_grad()
    for _ in range(3):
        gl, rl = m.train_step(dX, X.shape, dT, T.shape), float(ref.step(X, T))
        assert abs(gl - rl) <= 5e-4 * abs(rl), (gl, rl)
    m.close()


def test_host_api_errors(sess):
    from vtl_b200 import capi, host
    m = host.Model(sess)
    with pytest.raises(capi.VtlbError):
        m.linear(4)  # no input layer yet
    m.input([8])
    m.linear(4)
    x = sess.dev.zeros((2, 8)); t = sess.dev.zeros((2, 4))
    with pytest.raises(capi.VtlbError):
        m.train_step(x, (2, 8), t, (2, 4))  # no loss configured
    m.mse_loss()
    with pytest.raises(capi.VtlbError):
        m.train_step(x, (2, 8), t, (2, 4))  # no optimizer
    with pytest.raises(capi.VtlbError):
        m.train_step(x, (2, 7), t, (2, 4), update=False)  # wrong input width
    m.close()


@pytest.mark.parametrize("M,K,N", [(2, 2, 2), (96, 130, 50), (512, 300, 256)])
def test_variable_matmul_gate(sess, orc, M, K, N):
    """Variable.matmul / MatMulGate (autograd/variable_ops.v:82-94, gates_blas.v:41-46):
    C = A.B, dA = G.B^T, dB = A^T.G with G = C - T from the MSE loss."""
    rng = np.random.default_rng(M + K + N)
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    T = rng.standard_normal((M, N)).astype(np.float32)
    dA_, dB_, dT_ = (sess.dev.to_device(a) for a in (A, B, T))
    loss, C, dA, dB = sess.matmul_mse_backprop(dA_, M, K, dB_, N, dT_)
    rC = orc.matmul_f32(A, B)
    G = orc.mse_bwd_f32(rC, T)
    assert np.abs(C - rC).max() <= bound(K, A, B)
    assert abs(loss - float(orc.mse_f32(rC, T))) <= 1e-4 * float(orc.mse_f32(rC, T))
    assert np.abs(dA - orc.matmul_f32(G, B, tb=True)).max() <= bound(N, G, B) * 2
    assert np.abs(dB - orc.matmul_f32(A, G, ta=True)).max() <= bound(M, A, G) * 2
