"""Worker for tests/test_dist_cpu.py: runs under torch.distributed.run with the gloo backend
on CPU ranks and checks the host-side logic of the multi-GPU paths (rank plumbing, sharding,
the arithmetic identities data-parallel training and column-sharded INT8 inference rest on)
against the CPU oracle.  No GPU and no product kernel is involved."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402
import bench_train  # noqa: E402
from oracle import oracle  # noqa: E402


class FakeDevice:
    """Stands in for vtl_b200.capi.Device: records what the plumbing asks of it."""

    def __init__(self):
        self.calls = []

    def comm_unique_id(self):
        return bytes([7]) * 64 + os.urandom(64)

    def comm_init_rank(self, world, rank, uid):
        self.calls.append((world, rank, uid))

    def zeros(self, n, dtype=np.float32):
        return np.zeros(n, dtype)


def all_reduce_np(a, op):
    t = torch.from_numpy(np.ascontiguousarray(a))
    dist.all_reduce(t, op=op)
    return t.numpy()


def case_plumbing():
    ranks = bench.Ranks(int(os.environ["WORLD_SIZE"]))
    dev = FakeDevice()
    ranks.attach(dev)
    (world, rank, uid), = dev.calls
    assert world == ranks.world == 2 and rank == ranks.rank
    gathered = [None, None]
    dist.all_gather_object(gathered, uid)
    assert gathered[0] == gathered[1] and len(uid) == 128, "every rank must receive rank 0's id"
    ranks.barrier()
    ranks.close()


def case_dp_gradients():
    """Summing per-shard gradients (MSE gradient p - t has no 1/N; the loss divisor is the
    global element count) reproduces the full-batch gradient of the reference."""
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    wl = [bench_train.Workload("mlp_c1", world, r) for r in range(world)]
    me = wl[rank]
    assert me.global_rows == 64 * world and me.local_rows == 64
    p = me.params()
    for a, b in zip(p, wl[1 - rank].params()):
        assert np.array_equal(a, b), "replicas must start identical"
    X, T = me.batch()
    Xo, To = wl[1 - rank].batch()
    assert not np.array_equal(X, Xo), "ranks must see different rows"
    net = me.oracle_model(blas=False)
    _, y, dWs, dbs, _ = net.grads(X, T)
    part = float(((y.astype(np.float64) - T) ** 2).sum())
    loss = all_reduce_np(np.array([part]), dist.ReduceOp.SUM)[0] / (me.global_rows * 10)
    summed = [all_reduce_np(g, dist.ReduceOp.SUM) for g in dWs + dbs]
    # the same thing on the whole batch, on one rank
    order = [wl[r].batch() for r in range(world)]
    Xf, Tf = np.concatenate([o[0] for o in order]), np.concatenate([o[1] for o in order])
    full = me.oracle_model(blas=False)
    floss, _, fdWs, fdbs, _ = full.grads(Xf, Tf)
    assert abs(loss - float(floss)) <= 1e-5 * abs(float(floss))
    for s, f in zip(summed, fdWs + fdbs):
        assert np.abs(s - f).max() <= 1e-5 * max(1.0, float(np.abs(f).max()))
    dist.destroy_process_group()


def case_dp_accumulate():
    """Two backprops before an update, data-parallel: every backprop's bucket is all-reduced and the
    reduced gradients are then added on each rank (the host mirror orders that add after the
    collective).  Sum of reduced == reduced sum == twice the full-batch gradient, on every rank."""
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    wl = [bench_train.Workload("mlp_c1", world, r) for r in range(world)]
    me = wl[rank]
    X, T = me.batch()
    _, _, dWs, dbs, _ = me.oracle_model(blas=False).grads(X, T)
    acc = None
    for _ in range(2):  # backprop, all-reduce, accumulate
        red = [all_reduce_np(g.copy(), dist.ReduceOp.SUM) for g in dWs + dbs]
        acc = red if acc is None else [a + r for a, r in zip(acc, red)]
    order = [wl[r].batch() for r in range(world)]
    Xf, Tf = np.concatenate([o[0] for o in order]), np.concatenate([o[1] for o in order])
    _, _, fdWs, fdbs, _ = me.oracle_model(blas=False).grads(Xf, Tf)
    for a, f in zip(acc, fdWs + fdbs):
        assert np.abs(a - 2.0 * f).max() <= 2e-5 * max(1.0, float(np.abs(f).max()))
    # and the replicas hold the same accumulated gradient bit for bit
    for a in acc:
        other = [None, None]
        dist.all_gather_object(other, a.tobytes())
        assert other[0] == other[1]
    dist.destroy_process_group()


def case_int8_column_shards():
    """Column-sharded INT8 layers with a max all-reduce of the row maxima and an all-gather of
    the codes give the unsharded result bit for bit."""
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    rng = np.random.default_rng(11)  # same stream on every rank: full tensors, then slice
    M, dims = 48, [64, 128, 96]
    X = rng.standard_normal((M, dims[0])).astype(np.float32)
    Ws = [(rng.standard_normal((dims[i + 1], dims[i])) * 0.05).astype(np.float32) for i in range(2)]
    bs = [(rng.standard_normal(dims[i + 1]) * 0.01).astype(np.float32) for i in range(2)]
    ref = X
    for i in range(2):
        wq, sw = oracle.quant_rows_i8(Ws[i])
        ref = oracle.linear_i8_fwd(ref, wq, sw, bs[i], relu=(i == 0))
    aq, sa = oracle.quant_rows_i8(X)
    out = None
    for i in range(2):
        n = dims[i + 1] // world
        sl = slice(rank * n, (rank + 1) * n)
        wq, sw = oracle.quant_rows_i8(Ws[i][sl])
        acc = oracle.gemm_i8_i32(aq, wq)
        Y = oracle.dequant_bias_relu(acc, sa, sw, bs[i][sl], relu=(i == 0))
        if i == 1:
            out = Y
            break
        amax = all_reduce_np(np.abs(Y).max(axis=1).astype(np.float32), dist.ReduceOp.MAX)
        q, sa = oracle.quant_rows_i8_with_amax(Y, amax)
        parts = [torch.empty((M, n), dtype=torch.int8) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(q))
        aq = np.concatenate([p.numpy() for p in parts], axis=1)
    n = dims[2] // world
    assert np.array_equal(out.view(np.uint32), ref[:, rank * n:(rank + 1) * n].view(np.uint32))
    dist.destroy_process_group()


if __name__ == "__main__":
    {"plumbing": case_plumbing, "dp_gradients": case_dp_gradients, "dp_accumulate": case_dp_accumulate,
     "int8_column_shards": case_int8_column_shards}[sys.argv[1]]()
    print(f"rank {os.environ.get('RANK')} ok")
