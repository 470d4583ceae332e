"""Data-parallel plumbing of the host mirror on ONE GPU: a communicator of a single rank takes the
same code path as N ranks (gradient buckets all-reduced on the communication stream, the loss
all-reduced, the optimizer waiting for the collectives), and its collectives are identities, so
every result must equal the plain single-GPU session bit for bit.  Covers the orderings between
the compute and the communication stream: gradients accumulated over two backprops before an
update, frees of blocks that no collective touches, and the one-step weights of config 1."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def kaiming_uniform(rng, out_f, in_f):
    return (rng.uniform(-1, 1, (out_f, in_f)) * np.sqrt(6.0 / in_f)).astype(np.float32)


def make_session(with_comm):
    from vtl_b200 import capi, host
    if capi.device_count() == 0:
        pytest.skip("no CUDA device")
    s = host.Session(0)
    if with_comm:
        s.comm_init(1, 0, s.dev.comm_unique_id())
    return s


def build(sess, dims, relu_after, params, opt):
    from vtl_b200 import host
    m = host.Model(sess)
    m.input([dims[0]])
    for i, d in enumerate(dims[1:]):
        m.linear(d)
        if relu_after[i]:
            m.relu()
    m.mse_loss()
    (m.adamw if opt == "adamw" else m.adam)(lr=1e-3)
    for i, p in enumerate(params):
        m.set_param(i, p)
    return m


@pytest.mark.parametrize("small_limit", [0.0, 1.4e8])
@pytest.mark.parametrize("opt", ["adam", "adamw"])
def test_single_rank_communicator_equals_plain_session(opt, small_limit):
    rng = np.random.default_rng(21)
    dims, relu_after = [96, 160, 64, 32], [True, True, False]
    params = []
    for i in range(3):
        params += [kaiming_uniform(rng, dims[i + 1], dims[i]), (rng.standard_normal(dims[i + 1]) * 0.1).astype(np.float32)]
    X = rng.standard_normal((200, 96)).astype(np.float32)
    T = rng.standard_normal((200, 32)).astype(np.float32)
    results = []
    for with_comm in (False, True):
        s = make_session(with_comm)
        s.dev.set_small_gemm_limit(small_limit)
        m = build(s, dims, relu_after, params, opt)
        dX, dT = s.dev.to_device(X), s.dev.to_device(T)
        losses = []
        # two backprops before the first update: the second accumulates onto gradients whose
        # all-reduce was started by the first
        losses.append(m.train_step(dX, X.shape, dT, T.shape, global_rows=200, update=False))
        g_once = [m.get_grad(i) for i in range(6)]
        losses.append(m.train_step(dX, X.shape, dT, T.shape, global_rows=200, update=True))
        for _ in range(3):
            losses.append(m.train_step(dX, X.shape, dT, T.shape, global_rows=200))
        results.append((losses, g_once, [m.get_param(i) for i in range(6)], [m.get_moment(i) for i in range(6)]))
        assert s.dev.check_status() == 0
        m.close()
        s.close()
    (l0, g0, p0, m0), (l1, g1, p1, m1) = results
    assert l0 == l1
    for a, b in zip(g0 + p0 + m0, g1 + p1 + m1):
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_two_backprops_double_the_gradient():
    """parent.grad = parent.grad.add(diff) (autograd/variable.v:105) with all-reduces in flight:
    x + x is exact, so the accumulated gradient is exactly twice the single one."""
    rng = np.random.default_rng(22)
    dims, relu_after = [40, 24, 8], [True, False]
    params = [kaiming_uniform(rng, 24, 40), np.zeros(24, np.float32), kaiming_uniform(rng, 8, 24), np.zeros(8, np.float32)]
    X = rng.standard_normal((64, 40)).astype(np.float32)
    T = rng.standard_normal((64, 8)).astype(np.float32)
    s = make_session(True)
    m = build(s, dims, relu_after, params, "adam")
    dX, dT = s.dev.to_device(X), s.dev.to_device(T)
    m.train_step(dX, X.shape, dT, T.shape, update=False)
    once = [m.get_grad(i) for i in range(4)]
    m.train_step(dX, X.shape, dT, T.shape, update=False)
    twice = [m.get_grad(i) for i in range(4)]
    for a, b in zip(once, twice):
        assert np.array_equal(2.0 * a, b)
    assert s.dev.check_status() == 0
    m.close()
    s.close()


def test_config1_one_step_weights(orc):
    """Baseline config 1, ONE Adam step through the host mirror against the oracle.  The first Adam
    step moves every weight by lr * g / (|g| + eps') -- about lr in the direction of the gradient --
    so two implementations agree to rounding wherever the gradient is not within rounding of zero;
    where it is (|g| of the order of the GEMMs' own error), the step's direction is undetermined
    and the weights may differ by up to 2 * lr.  Checked: the bound 1e-5 * sqrt(K) * max|A| * max|B|
    of the gradient product on every weight whose oracle gradient exceeds that product's own
    error bound, and at most 2 * lr on the few that do not."""
    rng = np.random.default_rng(1)
    X = rng.random((64, 784), dtype=np.float32)
    T = np.eye(10, dtype=np.float32)[rng.integers(0, 10, 64)]
    W1, W2 = kaiming_uniform(rng, 256, 784), kaiming_uniform(rng, 10, 256)
    b1, b2 = np.zeros(256, np.float32), np.zeros(10, np.float32)
    s = make_session(False)
    for limit in (0.0, 1.4e8):  # tensor-core route and the default CUDA-core route of small products
        s.dev.set_small_gemm_limit(limit)
        m = build(s, [784, 256, 10], [True, False], [W1, b1, W2, b2], "adam")
        ref = orc.MLPOracle([W1, W2], [b1, b2], [True, False], lr=1e-3)
        _, y, dWs, dbs, _ = ref.grads(X, T)
        ref.step(X, T)
        dX, dT = s.dev.to_device(X), s.dev.to_device(T)
        m.train_step(dX, X.shape, dT, T.shape)
        g2 = y - T
        h = orc.relu_f32(orc.linear_fwd_f32(X, W1, b1))
        dhp = orc.relu_bwd_f32(orc.linear_bwd_f32(g2, h, W2)[0], orc.linear_fwd_f32(X, W1, b1))
        k = 1e-5 * np.sqrt(64.0)  # the contraction of every weight-gradient product runs over the 64 rows
        prod_bound = {0: k * np.abs(dhp).max() * np.abs(X).max(), 1: k * np.abs(dhp).max(),
                      2: k * np.abs(g2).max() * np.abs(h).max(), 3: k * np.abs(g2).max()}
        for i, (r, g) in enumerate(((ref.W[0], dWs[0]), (ref.b[0], dbs[0]), (ref.W[1], dWs[1]), (ref.b[1], dbs[1]))):
            diff = np.abs(m.get_param(i) - r.ravel())
            sure = np.abs(g.ravel()) > prod_bound[i]
            assert diff[sure].max() <= prod_bound[i], (i, diff[sure].max(), prod_bound[i])
            assert diff.max() <= 2.0e-3 + 1e-6, (i, diff.max())
            assert sure.mean() > 0.5  # the bound is checked on the bulk of the weights, not a remnant
        m.close()
    s.close()


def test_plane_passing_changes_no_bit():
    """The host mirror's large-layer path (operand planes handed from the producing product to the
    consuming ones, ReLU backward folded into the gradient product) against the plain path in which
    every product splits its own operands: losses, gradients, parameters and moments identical."""
    rng = np.random.default_rng(31)
    dims, relu_after = [128, 256, 192, 64], [True, True, False]
    params = []
    for i in range(3):
        params += [kaiming_uniform(rng, dims[i + 1], dims[i]), (rng.standard_normal(dims[i + 1]) * 0.1).astype(np.float32)]
    X = rng.standard_normal((320, 128)).astype(np.float32)
    T = rng.standard_normal((320, 64)).astype(np.float32)
    results = []
    for fuse_relu in (True, False):
        for on in (True, False):
            s = make_session(False)
            s.set_pass_planes(on)
            s.set_plane_min_flops(0.0)       # hand planes on at this size too
            s.dev.set_small_gemm_limit(0.0)  # all products large enough for the tensor-core path
            m = build(s, dims, relu_after, params, "adamw")
            m.set_fuse_relu(fuse_relu)
            dX, dT = s.dev.to_device(X), s.dev.to_device(T)
            loss0 = m.train_step(dX, X.shape, dT, T.shape, update=False)
            grads = [m.get_grad(i) for i in range(6)] + [m.input_grad(X.shape)]
            m.zero_grad()
            losses = [loss0] + [m.train_step(dX, X.shape, dT, T.shape) for _ in range(3)]
            results.append((losses, grads, [m.get_param(i) for i in range(6)]))
            assert s.dev.check_status() == 0
            m.close()
            s.close()
    base = results[-1]
    for losses, grads, ps in results[:-1]:
        assert losses == base[0]
        for a, b in zip(grads + ps, base[1] + base[2]):
            assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_shared_buffer_and_push_without_peers():
    """A buffer for the copy-engine all-gather comes back zeroed with a 64-byte handle; a push with
    no peer to write to is just the one-word all-reduce behind the compute stream; argument errors."""
    from vtl_b200 import capi
    dev = capi.Device(0)
    dev.comm_init_rank(1, 0, dev.comm_unique_id())
    ptr, handle = dev.shared_alloc(1 << 20)
    assert ptr and len(handle) == 64 and any(handle)
    back = np.empty(1 << 20, np.uint8)
    dev.d2h_raw(back.ctypes.data, ptr, back.nbytes)
    dev.sync()
    assert not back.any()
    src = dev.to_device(np.arange(4096, dtype=np.float32))
    dev.allgather_push_async(src, [None], 4096 * 4)
    dev.comm_mark(dev.LANE_BULK, 3)
    dev.comm_wait_mark(3)
    dev.comm_wait()
    dev.sync()
    assert np.array_equal(src.numpy(), np.arange(4096, dtype=np.float32))
    with pytest.raises(capi.VtlbError):
        dev.shared_alloc(0)
    assert dev.check_status() == 0
    dev.shared_free(ptr)
    dev.close()
