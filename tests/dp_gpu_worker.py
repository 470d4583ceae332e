"""Worker for tests/test_gpu_dp_multi.py: one process per GPU under torch.distributed.run.  Trains a
reduced config 4 data-parallel over all ranks through the C++ host mirror (NCCL all-reduce of the
gradient buckets on the communication stream) and checks it against rank 0 training alone on the
whole batch, then runs the column-sharded INT8 pipeline against the unsharded CPU oracle."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import bench  # noqa: E402
import bench_infer  # noqa: E402
import bench_train  # noqa: E402


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    ranks = bench.Ranks(int(os.environ["WORLD_SIZE"]))
    rep = bench_train.dp_matches_single_gpu(ranks, steps=3, width=256, layers=3, batch=1024)
    if ranks.rank == 0:
        assert rep["within_bound"], rep
        assert rep["loss_rel_diff"] <= 1e-5, rep
    # replicas agree bit for bit after training through the full session path
    from vtl_b200 import host
    session = host.Session(ranks.local_rank)
    ranks.attach(session.dev, session)
    wl = bench_train.Workload("mlp_c1", ranks.world, ranks.rank)
    model = wl.build(session)
    X, T = wl.batch()
    dX, dT = session.dev.to_device(X), session.dev.to_device(T)
    losses = [model.train_step(dX, X.shape, dT, T.shape, global_rows=wl.global_rows) for _ in range(5)]
    every = ranks.gather_objects(losses)
    assert all(l == every[0] for l in every), "the all-reduced loss must be the same number on every rank"
    agree = bench_train.replica_agreement(ranks, model)
    if ranks.rank == 0:
        assert agree == 0.0, agree
    assert session.dev.check_status() == 0
    model.close()
    session.close()
    # column-sharded INT8 inference over the same ranks
    from vtl_b200 import capi
    dev = capi.Device(ranks.local_rank)
    ranks.attach(dev)
    # the codes all-gathered by the copy engines (each rank copies into the peers' buffers), then
    # by NCCL's kernel; three layers make a buffer that is pushed into again within one pass
    for gather in ("push", "nccl"):
        os.environ["VTLB_C5_GATHER"] = gather
        W = ranks.world  # every shard must be a multiple of 128 columns wide
        for dims, chunks in (((256 * W, 512 * W, 256 * W), 2), ((128 * W, 256 * W, 128 * W, 256 * W, 128 * W), 4)):
            par = bench_infer.sharded_parity(ranks, dev, dims=dims, tokens=256, chunks=chunks)
            if ranks.rank == 0:
                assert par["bit_exact"], (gather, par)
    assert dev.check_status() == 0
    dev.close()
    ranks.close()
    print(f"rank {ranks.rank} ok")


if __name__ == "__main__":
    main()
