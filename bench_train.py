"""f32 training workloads of bench.py (`--workload mlp_c1 | mlp_c4 | cnn_c3`), run through
the C++ host mirror of vtl's Sequential / autograd / optimizer API (vtl_b200.host).

mlp_c1  baseline config 1: Sequential 784 -> 256 -> 10 (Linear, ReLU, Linear), batch 64,
        MSE vs one-hot targets, Adam lr 1e-3.  With N ranks every rank trains on 64 rows
        of a 64*N batch (weak scaling).
mlp_c4  baseline config 4: 8 Linear layers of width 4096 (ReLU after the first seven),
        global batch 65536 split evenly over the ranks (strong scaling), MSE vs N(0,1)
        targets, AdamW lr 1e-4 wd 0.01, gradient all-reduce (sum) per layer over NCCL,
        started during backprop and awaited before the optimizer step.
cnn_c3  baseline config 3: conv3x3 3->32 +ReLU, conv3x3 32->64 +ReLU, 2x2 max-pool,
        Linear 16384->10, softmax cross-entropy, Adam lr 1e-3, batch 256 split over ranks.

The metric is training samples per second (whole job).  `e2e` copies the step's batch and
targets from pinned host memory and reads the loss back every step."""
from __future__ import annotations

import ctypes as C
import statistics
import time

import numpy as np


def kaiming_uniform(rng, shape, fan_in):
    return (rng.uniform(-1.0, 1.0, shape) * np.sqrt(6.0 / fan_in)).astype(np.float32)


class Workload:
    def __init__(self, name, world, rank, rows=None):
        """`rows` (global batch) replaces the configuration's batch: only for small profiling
        captures, the result then says so in config.global_batch."""
        self.name, self.world, self.rank = name, world, rank
        self._init(name, world)
        if rows:
            self.global_rows = int(rows)
            self.local_rows = self.global_rows // world

    def _init(self, name, world):
        if name == "mlp_c1":
            self.dims, self.relu = [784, 256, 10], [True, False]
            self.local_rows, self.global_rows = 64, 64 * world
            self.scaling, self.opt, self.loss = "weak", ("adam", dict(lr=1e-3)), "mse"
            self.seed, self.default_steps = 1, 100
        elif name == "mlp_c4":
            self.dims, self.relu = [4096] * 9, [True] * 7 + [False]
            self.global_rows = 65536
            self.local_rows = self.global_rows // world
            self.scaling, self.loss = "strong", "mse"
            self.opt = ("adamw", dict(lr=1e-4, weight_decay=0.01))
            self.seed, self.default_steps = 4, 20
        elif name == "cnn_c3":
            self.global_rows = 256
            self.local_rows = self.global_rows // world
            self.scaling, self.opt, self.loss = "strong", ("adam", dict(lr=1e-3)), "sce"
            self.seed, self.default_steps = 3, 50
        else:
            raise SystemExit(f"unknown workload {name}")

    # ---- parameters: same seed on every rank => identical replicas
    def params(self):
        rng = np.random.default_rng(self.seed)
        if self.name == "cnn_c3":
            return [kaiming_uniform(rng, (32, 3, 3, 3), 27), np.zeros(32, np.float32),
                    kaiming_uniform(rng, (64, 32, 3, 3), 288), np.zeros(64, np.float32),
                    kaiming_uniform(rng, (10, 16384), 16384), np.zeros(10, np.float32)]
        out = []
        for i in range(len(self.dims) - 1):
            out += [kaiming_uniform(rng, (self.dims[i + 1], self.dims[i]), self.dims[i]),
                    np.zeros(self.dims[i + 1], np.float32)]
        return out

    def batch(self, rows=None):
        """This rank's shard of the synthetic batch (one fixed batch, reused every step)."""
        rows = self.local_rows if rows is None else rows
        rng = np.random.default_rng(self.seed * 1000 + 17 + self.rank)
        if self.name == "mlp_c1":
            X = rng.random((rows, 784), dtype=np.float32)
            T = np.eye(10, dtype=np.float32)[rng.integers(0, 10, rows)]
        elif self.name == "mlp_c4":
            X = rng.standard_normal((rows, 4096), dtype=np.float32)
            T = rng.standard_normal((rows, 4096), dtype=np.float32)
        else:
            X = rng.standard_normal((rows, 3, 32, 32), dtype=np.float32)
            T = np.eye(10, dtype=np.float32)[rng.integers(0, 10, rows)]
        return X, T

    def build(self, session):
        from vtl_b200 import host
        m = host.Model(session)
        if self.name == "cnn_c3":
            m.input([3, 32, 32])
            m.conv2d(3, 32, (3, 3), padding=(1, 1)); m.relu()
            m.conv2d(32, 64, (3, 3), padding=(1, 1)); m.relu()
            m.maxpool2d((2, 2), (0, 0), (2, 2))
            m.flatten()
            m.linear(10)
            m.softmax_cross_entropy_loss()
        else:
            m.input([self.dims[0]])
            for i, d in enumerate(self.dims[1:]):
                m.linear(d)
                if self.relu[i]:
                    m.relu()
            m.mse_loss()
        kind, kw = self.opt
        (m.adam if kind == "adam" else m.adamw)(**kw)
        for i, p in enumerate(self.params()):
            m.set_param(i, p)
        return m

    def flops_per_step(self, rows):
        """Algorithmic FLOPs of forward + backward for `rows` samples (2*M*N*K per GEMM; dX of
        the first layer included, as the reference computes it)."""
        if self.name == "cnn_c3":
            conv = lambda C_, O: 2.0 * rows * 32 * 32 * O * C_ * 9
            lin = 2.0 * rows * 16384 * 10
            return 3.0 * (conv(3, 32) + conv(32, 64) + lin)
        return 3.0 * sum(2.0 * rows * self.dims[i] * self.dims[i + 1] for i in range(len(self.dims) - 1))

    def describe(self):
        if self.name == "mlp_c1":
            return ("f32 Sequential MLP 784->256->10 (Linear, ReLU, Linear), batch 64 per GPU, MSE vs "
                    "one-hot targets, Adam lr=1e-3 (baseline config 1)")
        if self.name == "mlp_c4":
            return ("f32 deep MLP, 8 Linear layers of width 4096 with ReLU (none after the last), global "
                    "batch 65536, MSE vs N(0,1) targets, AdamW lr=1e-4 wd=0.01 (baseline config 4)")
        return ("f32 CNN on CIFAR-shaped synthetic data: conv3x3 3->32+ReLU, conv3x3 32->64+ReLU, 2x2 "
                "max-pool, Linear 16384->10, softmax-CE, Adam lr=1e-3, batch 256 (baseline config 3)")

    # ---- the CPU oracle for this workload (reference arm / cpu_baseline)
    def oracle_model(self, blas=True):
        from oracle import oracle
        p = self.params()
        if self.name == "cnn_c3":
            return oracle.SequentialOracle(
                [("conv2d", p[0], p[1], (1, 1), (1, 1)), ("relu",), ("conv2d", p[2], p[3], (1, 1), (1, 1)),
                 ("relu",), ("maxpool2d", (2, 2), (0, 0), (2, 2)), ("flatten",), ("linear", p[4], p[5])],
                loss="sce", lr=1e-3, blas=blas)
        kind, kw = self.opt
        return oracle.MLPOracle(p[0::2], p[1::2], self.relu, lr=kw["lr"],
                                weight_decay=kw.get("weight_decay") if kind == "adamw" else None, blas=blas)

    def cpu_sample_rows(self):
        return {"mlp_c1": 64, "mlp_c4": 512, "cnn_c3": 8}[self.name]


def cpu_baseline(wl, steps=None, budget_s=15.0):
    """Times the CPU oracle (f32->f64 OpenBLAS dgemm GEMMs, scalar optimizer loops, direct conv
    loops) on a bounded sample of the workload; returns the cpu_baseline object."""
    from oracle import oracle
    oracle.build()
    rows = wl.cpu_sample_rows()
    X, T = wl.batch(rows)
    net = wl.oracle_model(blas=True)
    net.step(X, T)  # warm-up (BLAS threads, page faults)
    n, t0 = 0, time.perf_counter()
    while n < (steps or 10 ** 9) and (n == 0 or time.perf_counter() - t0 < budget_s):
        net.step(X, T)
        n += 1
        if steps is None and wl.name == "mlp_c1" and n >= 100:
            break
    dt = (time.perf_counter() - t0) / n
    import os
    return {"value": rows / dt, "unit": "samples/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{n} full training steps on a batch of {rows} rows (of {wl.global_rows}); GEMMs as "
                      f"f32->f64 OpenBLAS dgemm on all cores, optimizer and conv loops single-threaded C",
            "ms_per_step": dt * 1e3}, rows, dt


def run_reference(args, ranks):
    if ranks.rank != 0:
        return None
    wl = Workload(args.workload, 1, 0)
    cb, rows, dt = cpu_baseline(wl, steps=max(1, args.steps), budget_s=120.0)
    out = {"impl": "reference", "metric": "f32_train_samples_per_s", "value": cb["value"], "unit": "samples/s",
           "n_gpus": ranks.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
           "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None, "dtype": "f32 (f64 accumulate)",
           "data": "synthetic", "config": {"workload": wl.describe(), "rows_per_step": rows},
           "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
           "e2e": {"value": cb["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    return out


def run(args, ranks, ClockSampler, peaks, cuda_sync):
    from vtl_b200 import host
    wl = Workload(args.workload, ranks.world, ranks.rank, getattr(args, "rows", None))
    session = host.Session(ranks.local_rank)
    dev = session.dev
    ranks.attach(dev, session)  # the session creates the communicator, so its gates know the world size
    model = wl.build(session)
    X, T = wl.batch()
    dX, dT = dev.to_device(X), dev.to_device(T)
    xs, ts, G = X.shape, T.shape, wl.global_rows

    def step(want_loss=False):
        return model.train_step(dX, xs, dT, ts, global_rows=G, update=True, want_loss=want_loss)

    cuda_sync(dev)  # also pays the one-off import costs now, not between warm-up and timing
    sampler = ClockSampler(ranks.local_rank)
    if ranks.rank == 0:
        sampler.start()
    ranks.barrier()
    for _ in range(args.warmup):  # directly before the timed region: the GPU must not idle
        step()                    # (and drop its clocks) between warm-up and timing
    dev.sync()
    ranks.barrier()
    l0 = dev.launch_count()
    e0, e1 = dev.event(), dev.event()
    dev.record(e0)
    for _ in range(args.steps):
        step()
    dev.record(e1)
    ms_total = dev.elapsed_ms(e0, e1)
    launches = dev.launch_count() - l0
    cuda_sync(dev)
    ranks.barrier()
    ms_total = ranks.max_f32(ms_total)
    last_loss = step(want_loss=True)

    # the tensor-core GEMM launches alone, timed with event pairs around each launch
    prof_steps = max(1, min(args.steps, 2048 // 64))
    dev.profile_gemm(True)
    for _ in range(prof_steps):
        step()
    gemm_ms, gemm_n, gemm_ops = dev.profile_gemm_read()
    dev.profile_gemm(False)

    # end to end: batch and targets come from pinned host memory, the loss goes back, every step
    hX, hT = C.c_void_p(), C.c_void_p()
    assert dev.lib.vtlb_host_alloc(X.nbytes, C.byref(hX)) == 0
    assert dev.lib.vtlb_host_alloc(T.nbytes, C.byref(hT)) == 0
    C.memmove(hX.value, X.ctypes.data, X.nbytes)
    C.memmove(hT.value, T.ctypes.data, T.nbytes)

    # every step's batch and targets come from pinned host memory; the copy of the next batch runs on
    # the library's copy stream while the current step trains (two device buffers per input)
    dXs, dTs = [dX, dev.empty(X.shape, X.dtype)], [dT, dev.empty(T.shape, T.dtype)]

    def e2e_run(steps):
        dev.copy_h2d_async(dXs[0], hX.value, X.nbytes)
        dev.copy_h2d_async(dTs[0], hT.value, T.nbytes)
        loss = None
        for i in range(steps):
            dev.copy_wait(dev.COPY_IN_BEFORE_COMPUTE)
            if i + 1 < steps:
                dev.copy_h2d_async(dXs[(i + 1) % 2], hX.value, X.nbytes)
                dev.copy_h2d_async(dTs[(i + 1) % 2], hT.value, T.nbytes)
            loss = model.train_step(dXs[i % 2], xs, dTs[i % 2], ts, global_rows=G, update=True, want_loss=True)
        return loss

    e2e_run(2)
    cuda_sync(dev)
    ranks.barrier()
    e2e_steps = max(1, min(args.steps, 20))
    t0 = time.perf_counter()
    e2e_run(e2e_steps)
    cuda_sync(dev)
    e2e_ms = ranks.max_f32((time.perf_counter() - t0) * 1e3)
    clocks = sampler.stop() if ranks.rank == 0 else None
    assert dev.check_status() == 0
    dev.lib.vtlb_host_free(hX)
    dev.lib.vtlb_host_free(hT)

    out = None
    if ranks.rank == 0:
        pk = peaks()
        ms_step = ms_total / args.steps
        # GEMMs timed inside a step that keeps the GPU busy for hundreds of ms run under the power
        # cap: the sustained figure is the yardstick there, the burst figure for short steps
        long_step = ms_step > 50.0
        bf16_peak = pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) if long_step else pk["bf16_tflops"]
        tf32x3_peak = bf16_peak / 2.0 / 3.0
        gemm_tflops = gemm_ops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        out = {
            "metric": "f32_train_samples_per_s", "value": G / (ms_step * 1e-3), "unit": "samples/s",
            "n_gpus": ranks.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None,
            "dtype": "f32 (3xTF32 tensor-core products, f32 accumulate)", "data": "synthetic",
            "config": {"workload": wl.describe(), "global_batch": G, "rows_per_gpu": wl.local_rows,
                       "parallelism": f"dp{ranks.world}: batch rows sharded, per-layer NCCL all-reduce(sum) of "
                                      "gradients overlapped with backprop" if ranks.world > 1 else "single GPU",
                       "l2": "activations and gradients of a step exceed the 126 MB L2" if wl.name != "mlp_c1"
                             else "working set (1.7 MB) fits in L2: the step is launch-latency bound; no flush",
                       "final_loss": last_loss,
                       "algorithmic_tflops_per_s": wl.flops_per_step(G) / (ms_step * 1e-3) / 1e12},
            "e2e": {"value": G / (e2e_ms / e2e_steps * 1e-3), "unit": "samples/s",
                    "h2d_bytes_per_step": int(X.nbytes + T.nbytes), "d2h_bytes_per_step": 4,
                    "ms_per_step": e2e_ms / e2e_steps},
            "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "gemm_tc_kernel<tf32 x3> (all GEMM launches of a step)",
                         "achieved": gemm_tflops, "peak": tf32x3_peak, "unit": "TFLOP/s",
                         "frac": (gemm_tflops / tf32x3_peak) if gemm_tflops else None, "traffic": None,
                         "peak_source": f"{'bf16_tflops_sustained' if long_step else 'bf16_tflops'} of "
                                        f"{pk['_source']} / 2 (TF32 rate) / 3 (three MMAs per algorithmic product)",
                         "kernel_ms_per_step": gemm_ms / prof_steps, "launches_per_step": gemm_n / prof_steps},
        }
        if ranks.world == 1:
            cb, _, _ = cpu_baseline(wl)
            out["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    model.close()
    session.close()
    return out


# ------------------------------------------------------------------ config 4 inside the default bench line
def _bcast_params_from_last(ranks, params):
    """Rank N-1's parameter arrays on rank 0 (control plane, gloo point to point); None elsewhere."""
    import torch
    dist, last = ranks.dist, ranks.world - 1
    if ranks.rank == last:
        for p in params:
            dist.send(torch.from_numpy(np.ascontiguousarray(p)), dst=0)
        return None
    if ranks.rank == 0:
        out = []
        for p in params:
            buf = torch.empty(p.shape, dtype=torch.float32)
            dist.recv(buf, src=last)
            out.append(buf.numpy())
        return out
    return None


def replica_agreement(ranks, model):
    """max |theta(rank 0) - theta(rank N-1)| over every parameter tensor.  The replicas start from
    the same weights, add up the same all-reduced gradients and run the same optimizer kernel, so
    anything but 0 is a bug.  Rank 0 returns the number, the others None."""
    if ranks.world == 1:
        return 0.0
    mine = [model.get_param(i) for i in range(model.num_params())] if ranks.rank in (0, ranks.world - 1) else []
    theirs = _bcast_params_from_last(ranks, mine)
    ranks.barrier()
    if ranks.rank != 0:
        return None
    return float(max(np.abs(a - b).max() for a, b in zip(mine, theirs)))


def dp_matches_single_gpu(ranks, steps=3, width=512, layers=4, batch=4096):
    """A reduced config 4 (4 Linear layers of width 512 with ReLU between, batch 4096, MSE, AdamW)
    trained for `steps` steps (a) data-parallel over all ranks and (b) by rank 0 alone on the whole
    batch, from the same weights.  The two runs differ only in the order in which the rows of the
    batch are summed into dW and db, so the parameters must agree within the bound of the
    weight-gradient product, 1e-5 * sqrt(K) * max|A| * max|B| with K = batch rows, A the loss
    gradient P - T and B the layer inputs, taken at their largest over the layers.  Rank 0 returns
    the report, the others None."""
    from vtl_b200 import host
    dims, relu = [width] * (layers + 1), [True] * (layers - 1) + [False]
    rng = np.random.default_rng(44)
    params = []
    for i in range(layers):
        params += [kaiming_uniform(rng, (dims[i + 1], dims[i]), dims[i]), np.zeros(dims[i + 1], np.float32)]
    X = rng.standard_normal((batch, width), dtype=np.float32)
    T = rng.standard_normal((batch, width), dtype=np.float32)

    def build(session):
        m = host.Model(session)
        m.input([width])
        for i in range(layers):
            m.linear(width)
            if relu[i]:
                m.relu()
        m.mse_loss()
        m.adamw(lr=1e-4, weight_decay=0.01)
        for i, p in enumerate(params):
            m.set_param(i, p)
        return m

    def train(session, Xs, Ts):
        m = build(session)
        dX, dT = session.dev.to_device(Xs), session.dev.to_device(Ts)
        losses = [m.train_step(dX, Xs.shape, dT, Ts.shape, global_rows=batch) for _ in range(steps)]
        out = [m.get_param(i) for i in range(2 * layers)]
        dX.free(); dT.free()
        m.close()
        return losses, out

    # (a) all ranks, each on its rows
    per = batch // ranks.world
    sa = host.Session(ranks.local_rank)
    if ranks.world > 1:
        box = [sa.dev.comm_unique_id() if ranks.rank == 0 else None]
        ranks.dist.broadcast_object_list(box, src=0)
        sa.comm_init(ranks.world, ranks.rank, box[0])
    lo = ranks.rank * per
    dp_losses, dp_params = train(sa, X[lo:lo + per], T[lo:lo + per])
    assert sa.dev.check_status() == 0
    sa.close()
    ranks.barrier()
    if ranks.rank != 0:
        return None
    # (b) rank 0 alone on the whole batch (no communicator)
    sb = host.Session(ranks.local_rank)
    one_losses, one_params = train(sb, X, T)
    sb.close()
    # bound of the weight-gradient products: K = batch rows; |P - T| and the layer inputs at step 0
    acts, amax_in, a = X, float(np.abs(X).max()), X
    for i in range(layers):
        a = a @ params[2 * i].T + params[2 * i + 1]
        if relu[i]:
            a = np.maximum(a, 0)
            amax_in = max(amax_in, float(np.abs(a).max()))
    gmax = float(np.abs(a - T).max())
    bound = 1e-5 * np.sqrt(batch) * gmax * amax_in
    diff = float(max(np.abs(p - q).max() for p, q in zip(dp_params, one_params)))
    return {"config": f"{layers} x Linear({width}) + ReLU, batch {batch}, MSE, AdamW, {steps} steps",
            "max_abs_param_diff_vs_one_gpu": diff, "bound": float(bound), "within_bound": bool(diff <= bound),
            "loss_dp": dp_losses, "loss_one_gpu": one_losses,
            "loss_rel_diff": float(max(abs(x - y) / abs(y) for x, y in zip(dp_losses, one_losses)))}


def run_dp(ranks, tools, steps=8, warmup=3):
    """Baseline config 4 on the ranks of this job (global batch 65536 split by rows, strong scaling):
    samples/s, the time of the tensor-core GEMMs inside a step, a breakdown of the rest of the step
    by phase, and the parity checks of the data-parallel path.  Returns the object on rank 0."""
    from vtl_b200 import host
    wl = Workload("mlp_c4", ranks.world, ranks.rank)
    session = host.Session(ranks.local_rank)
    dev = session.dev
    ranks.attach(dev, session)
    model = wl.build(session)
    X, T = wl.batch()
    dX, dT = dev.to_device(X), dev.to_device(T)
    xs, ts, G = X.shape, T.shape, wl.global_rows
    del X, T

    def run_steps(n):
        for _ in range(n):
            model.train_step(dX, xs, dT, ts, global_rows=G, update=True, want_loss=False)

    tools.cuda_sync(dev)
    ranks.barrier()
    run_steps(warmup)
    l0 = dev.launch_count()
    per_step, steps_per_repeat = tools.timed_repeats(dev, ranks, run_steps, steps, max_total_s=12.0)
    launches = dev.launch_count() - l0
    ms_step = statistics.median(per_step)
    # one more step for the loss value: the sum over the ranks' rows (all-reduced), over the global divisor
    loss = model.train_step(dX, xs, dT, ts, global_rows=G, update=True, want_loss=True)
    losses = ranks.gather_objects(loss)
    # phases of a step, each bracketed by CUDA events on the compute stream
    prof_steps = 2
    dev.profile_gemm(True)
    run_steps(prof_steps)
    phases = dev.profile_read_phases()
    gemm_ms, gemm_n, gemm_ops = dev.profile_gemm_read()
    dev.profile_gemm(False)
    agree = replica_agreement(ranks, model)
    assert dev.check_status() == 0
    model.close()
    dX.free(); dT.free()
    session.close()
    small = dp_matches_single_gpu(ranks)
    if ranks.rank != 0:
        return None
    pk = tools.peaks()
    long_step = ms_step > 50.0
    bf16_peak = pk.get("bf16_tflops_sustained", pk["bf16_tflops"]) if long_step else pk["bf16_tflops"]
    tf32x3_peak = bf16_peak / 2.0 / 3.0
    gemm_tflops = gemm_ops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    ph = {k: v[0] / prof_steps for k, v in phases.items()}
    accounted = sum(ph.values())
    return {
        "workload": wl.describe(), "metric": "f32_train_samples_per_s", "value": G / (ms_step * 1e-3),
        "unit": "samples/s", "scaling": "strong", "global_batch": G, "rows_per_gpu": wl.local_rows,
        "ms_per_step": ms_step, "timing": dict(tools.spread(per_step), steps_per_repeat=steps_per_repeat),
        "gpu_launches": int(launches),
        "gemm_ms_per_step": gemm_ms / prof_steps, "gemm_launches_per_step": gemm_n / prof_steps,
        "gemm_tflops": gemm_tflops, "gemm_frac_of_peak": gemm_tflops / tf32x3_peak if gemm_tflops else None,
        "gemm_peak": tf32x3_peak,
        "gemm_peak_source": f"{'bf16_tflops_sustained' if long_step else 'bf16_tflops'} of {pk['_source']} / 2 "
                            "(TF32 rate) / 3 (three MMAs per algorithmic product)",
        "phases_ms_per_step": {"gemm": ph["gemm"], "operand_split": ph["operand_split"], "optimizer": ph["optimizer"],
                               "elementwise": ph["elementwise"], "exposed_allreduce_wait": ph["comm_wait"],
                               "everything_else": max(0.0, ms_step - accounted),
                               "note": "CUDA-event brackets on the compute stream over two profiled steps; "
                                       "exposed_allreduce_wait is the time the compute stream stood idle before "
                                       "the optimizer until the gradient all-reduces had finished"},
        "parallelism": (f"dp{ranks.world}: batch rows sharded, one NCCL all-reduce(sum) per layer (dW and db in one "
                        "bucket) on a communication stream, started as the layer's backward finishes; AdamW after the "
                        "last one") if ranks.world > 1 else "single GPU",
        "parity": {"loss": loss, "loss_is_global": "sum over the ranks' rows / global element count, all-reduced",
                   "loss_equal_on_all_ranks": bool(all(x == losses[0] for x in losses)),
                   "max_abs_param_diff_rank0_vs_last": agree,
                   "dp_vs_one_gpu_reduced_config": small},
    }
