"""Output-column-sharded INT8 MLP inference, emulated on one GPU: R "ranks" run one after the
other, the row-max all-reduce and the all-gather of codes are done by hand, and the result
must equal the unsharded oracle bit for bit (max is associative, quantisation is
element-wise, the int32 GEMM is exact)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def oracle_mlp(orc, X, Ws, bs):
    A = X
    for i, (W, b) in enumerate(zip(Ws, bs)):
        wq, sw = orc.quant_rows_i8(W)
        A = orc.linear_i8_fwd(A, wq, sw, b, relu=(i + 1 < len(Ws)))
    return A


@pytest.mark.parametrize("M,dims,R", [(300, [512, 1024, 512], 4), (640, [256, 512, 768, 256], 2)])
def test_sharded_int8_mlp_bit_exact(dev, orc, M, dims, R):
    rng = np.random.default_rng(M + R)
    X = rng.standard_normal((M, dims[0])).astype(np.float32)
    Ws = [(rng.standard_normal((dims[i + 1], dims[i])) * 0.05).astype(np.float32) for i in range(len(dims) - 1)]
    bs = [(rng.standard_normal(dims[i + 1]) * 0.01).astype(np.float32) for i in range(len(dims) - 1)]
    ref = oracle_mlp(orc, X, Ws, bs)

    # per-rank weight shards, quantised once
    shards = []
    for W, b in zip(Ws, bs):
        n = W.shape[0] // R
        per = []
        for r in range(R):
            dW = dev.to_device(W[r * n:(r + 1) * n])
            dQ, dS = dev.zeros((n, W.shape[1]), np.int8), dev.zeros(n)
            dev.quant_rows_i8(dW, n, W.shape[1], dQ, dS)
            per.append((dQ, dS, dev.to_device(b[r * n:(r + 1) * n])))
        shards.append(per)

    # layer 0 input: every rank quantises the replicated activations (one shard = plain layout)
    K = dims[0]
    dX = dev.to_device(X)
    dAq, dSa = dev.zeros((M, K), np.int8), dev.zeros(M)
    dev.quant_rows_i8(dX, M, K, dAq, dSa)
    a_shards = 1
    out = None
    for li in range(len(Ws)):
        N, K = Ws[li].shape
        n = N // R
        last = li + 1 == len(Ws)
        slabs, amaxes = [], []
        for r in range(R):
            dQ, dS, db = shards[li][r]
            dY = dev.zeros((M, n))
            dev.linear_i8_fwd_sharded_a(dAq, a_shards, dSa, dQ, dS, db, dY, M, n, K, relu=not last)
            assert dev.check_status() == 0
            slabs.append(dY)
            if not last:
                dA = dev.zeros(M)
                dev.row_absmax_f32(dY, M, n, dA)
                amaxes.append(dA.numpy())
        if last:
            out = np.concatenate([s.numpy() for s in slabs], axis=1)
            break
        amax = dev.to_device(np.max(np.stack(amaxes), axis=0))  # the all-reduce(max) over ranks
        gathered = dev.zeros((R, M, n), np.int8)                # the all-gather of the code slabs
        dSa = dev.zeros(M)
        for r in range(R):
            dev.quant_rows_i8(slabs[r], M, n, gathered.ptr + r * M * n, dSa, amax)
        dAq, a_shards = gathered, R
    assert np.array_equal(out.view(np.uint32), ref.view(np.uint32)), np.abs(out - ref).max()


def test_sharded_a_argument_errors(dev):
    from vtl_b200.capi import VtlbError
    q = dev.zeros((64, 256), np.int8)
    s = dev.zeros(256)
    y = dev.zeros((64, 64))
    with pytest.raises(VtlbError):
        dev.linear_i8_fwd_sharded_a(q, 3, s, q, s, None, y, 64, 64, 256)   # 256 does not split in 3
    with pytest.raises(VtlbError):
        dev.linear_i8_fwd_sharded_a(q, 4, s, q, s, None, y, 64, 64, 256)   # shards of 64 columns


def test_row_block_pipeline_of_the_benchmark_model(dev, orc):
    """bench_infer.ShardedInt8MLP walks the tokens as independent row blocks (that is what lets
    the all-gather of one block overlap the GEMM of the next on several GPUs).  One rank, four
    blocks: same result as the oracle run on all rows at once."""
    import bench_infer
    dims, tokens, seed = [256, 512, 256], 512, 5
    model = bench_infer.ShardedInt8MLP(dev, 1, 0, tokens=tokens, dims=dims, seed=seed, chunks=4)
    X = np.random.default_rng(9).standard_normal((tokens, dims[0])).astype(np.float32)
    dX = dev.to_device(X)
    y = model.forward(dX)
    dev.sync()
    assert dev.check_status() == 0
    Ws, bs = [], []
    for li in range(len(dims) - 1):
        rng = np.random.default_rng([seed, li, 0])
        Ws.append(rng.standard_normal((dims[li + 1], dims[li]), dtype=np.float32) * np.float32(0.02))
        bs.append(rng.standard_normal(dims[li + 1], dtype=np.float32) * np.float32(0.01))
    ref = oracle_mlp(orc, X, Ws, bs)
    assert np.array_equal(y.numpy().view(np.uint32), ref.view(np.uint32))
