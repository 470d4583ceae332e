#!/usr/bin/env python
"""Benchmark of the dense-contraction hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload int8_linear|mlp_c1|mlp_c4]

Prints ONE JSON line on rank 0.  The default workload is the INT8 quantised
Linear forward at M = N = K = 4096: one step = per-row dynamic quantisation of the
f32 activations + int8 x int8 -> int32 GEMM on tcgen05 with the fused
dequant + bias + ReLU epilogue, against pre-quantised weights.  With N > 1 ranks
(one process per GPU, launched by torch.distributed.run) the layer is sharded by
output columns: every rank owns 4096 output channels of a 4096*N-wide layer and
the activations are replicated, so per-GPU work is fixed (weak scaling) and the
data path needs no collective.

`value` is whole-job throughput with operands resident in HBM; `e2e` is the same
step called with HOST buffers (pinned), including the host->device copy of the
activations and the device->host copy of the result.
`--impl reference` times the CPU oracle (oracle/, the restatement of the
reference's CPU arithmetic; the reference itself is V code plus an un-vendored
BLAS module and cannot be built here) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

I8_M = I8_N = I8_K = 4096
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        d["_source"] = "measured"
        return d
    d = dict(FALLBACK_PEAKS)
    d["_source"] = "fallback"
    return d


# ------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples the SM clock and the throttle reasons through NVML every few milliseconds
    while the timed regions run (reading only; no setting is changed)."""

    def __init__(self, gpu_index: int):
        self.gpu, self.samples, self.stop_flag, self.err = gpu_index, [], False, None
        self.thread = None

    def start(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            self.nv = nv
            self.h = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self.smax = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
        except Exception as e:  # NVML missing: report it, do not fail the benchmark
            self.err = f"nvml unavailable: {e}"
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def _loop(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                clk = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                rs = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                util = nv.nvmlDeviceGetUtilizationRates(self.h).gpu
                self.samples.append((clk, rs, util))
            except Exception as e:
                self.err = str(e)
                return
            time.sleep(0.005)

    def stop(self):
        self.stop_flag = True
        if self.thread:
            self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": [self.err or "no samples"]}
        nv = self.nv
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        reasons = sorted(k for k, bit in names.items() if any(s[1] & bit for s in self.samples))
        # clocks idle low between kernels: the figure that matters is the clock under load
        top = sorted(s[0] for s in self.samples)
        return {"sm_mhz": statistics.median(top), "sm_mhz_p90": top[int(0.9 * (len(top) - 1))],
                "sm_max_mhz": self.smax, "samples": len(top), "reasons": reasons}


# ------------------------------------------------------------------ distributed plumbing
class Ranks:
    """RANK / WORLD_SIZE from torchrun; a gloo group carries control messages (the NCCL
    unique id); timing reductions and data-path collectives go through the library's own
    NCCL communicator."""

    def __init__(self, want_gpus: int):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        # NCCL writes its version / debug lines to stdout when NCCL_DEBUG is set; stdout must
        # carry exactly one JSON line, so send them to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        if self.world > 1:
            import torch.distributed as dist
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            dist.init_process_group("gloo")
            self.dist = dist
        elif want_gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run "
                             "(one process per GPU)")

    def attach(self, dev, session=None):
        """Creates the NCCL communicator of this rank's context (through the host-mirror session
        when there is one, so that its gradient gates know the world size)."""
        self.dev = dev
        if self.world > 1:
            box = [dev.comm_unique_id() if self.rank == 0 else None]
            self.dist.broadcast_object_list(box, src=0)
            if session is not None:
                session.comm_init(self.world, self.rank, box[0])
            else:
                dev.comm_init_rank(self.world, self.rank, box[0])
            self._red = dev.zeros(4, np.float32)

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max_f32(self, x: float) -> float:
        if self.world == 1:
            return x
        dev = self.dev
        dev.h2d_raw(self._red, np.array([x, 0, 0, 0], np.float32).ctypes.data, 16)
        dev.sync()
        dev.allreduce_max_f32_async(self._red, 4)
        dev.comm_wait()
        return float(self._red.numpy()[0])

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def cuda_sync(dev):
    dev.sync()
    try:
        import torch
        if torch.cuda.is_available() and torch.cuda.is_initialized():
            torch.cuda.synchronize()
    except Exception:
        pass


# ------------------------------------------------------------------ INT8 workload
def make_int8_inputs(seed: int, rank: int, M: int = I8_M):
    """Config 2 of the baseline: A ~ N(0,1) [M,4096] (same on every rank; M = 4096 unless the
    run is one point of the config's M sweep), this rank's W shard ~ N(0,0.02) [4096,4096],
    bias ~ N(0,0.01) [4096]."""
    A = np.random.default_rng(seed).standard_normal((M, I8_K), dtype=np.float32)
    r = np.random.default_rng(seed + 1000 + rank)
    W = (r.standard_normal((I8_N, I8_K), dtype=np.float32) * np.float32(0.02))
    b = (r.standard_normal(I8_N, dtype=np.float32) * np.float32(0.01))
    return A, W, b


def cpu_int8_sample(A, W, b, budget_s=12.0):
    """Times the oracle's quantised linear forward on the first rows of A; returns
    (TOPS, threads, description)."""
    from oracle import oracle
    oracle.build()
    wq, sw = oracle.quant_rows_i8(W)
    M = A.shape[0]
    rows = min(32, M)
    t0 = time.perf_counter()
    oracle.linear_i8_fwd(A[:rows], wq, sw, b, True)
    dt = time.perf_counter() - t0
    rows = int(max(32, min(M, rows * budget_s / max(dt, 1e-3))))
    rows -= rows % 32
    rows = max(1, min(rows, M))
    reps, t0 = 0, time.perf_counter()
    while reps == 0 or time.perf_counter() - t0 < 0.8 * budget_s:
        oracle.linear_i8_fwd(A[:rows], wq, sw, b, True)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    tops = 2.0 * rows * I8_N * I8_K / dt / 1e12
    return (tops, oracle.max_threads(), f"first {rows} of {M} rows of A against all {I8_N} "
            f"channels, {reps} repeats, {dt * reps:.1f} s in total", rows, dt)


def run_int8(args, ranks):
    from vtl_b200 import capi
    dev = capi.Device(ranks.local_rank)
    ranks.attach(dev)
    M, N, K = (args.rows or I8_M), I8_N, I8_K
    A, W, b = make_int8_inputs(2, ranks.rank, M)
    # operand copies rotated between steps so that no step finds its operands in the 126 MB L2:
    # 4 x 160 MiB at M = 4096; with few rows a set is little more than the 16 MiB of weight codes
    set_bytes = M * K * 5 + M * N * 4 + N * K
    NSETS = max(4, -(-170_000_000 // set_bytes))
    dA = [dev.to_device(A) for _ in range(NSETS)]
    dQa = [dev.zeros((M, K), np.int8) for _ in range(NSETS)]
    dSa = [dev.zeros(M) for _ in range(NSETS)]
    dY = [dev.zeros((M, N)) for _ in range(NSETS)]
    dW = dev.to_device(W)
    dQw = [dev.zeros((N, K), np.int8) for _ in range(NSETS)]
    dSw = [dev.zeros(N) for _ in range(NSETS)]
    db = dev.to_device(b)
    for i in range(NSETS):  # weights are quantised once, ahead of time
        dev.quant_rows_i8(dW, N, K, dQw[i], dSw[i])
    dev.sync()

    def step(i):
        s = i % NSETS
        dev.quant_rows_i8(dA[s], M, K, dQa[s], dSa[s])
        dev.linear_i8_fwd(dQa[s], dSa[s], dQw[s], dSw[s], db, dY[s], M, N, K, True)

    cuda_sync(dev)  # also pays the one-off import costs now, not between warm-up and timing
    sampler = ClockSampler(ranks.local_rank)
    if ranks.rank == 0:
        sampler.start()  # keeps sampling through all three timed passes below
    ranks.barrier()
    for i in range(args.warmup):  # directly before the timed region: the GPU must not idle
        step(i)                   # (and drop its clocks) between warm-up and timing
    dev.sync()
    ranks.barrier()
    # pass 1: whole steps, one event pair around the timed region
    l0 = dev.launch_count()
    e0, e1 = dev.event(), dev.event()
    dev.record(e0)
    for i in range(args.steps):
        step(i)
    dev.record(e1)
    ms_total = dev.elapsed_ms(e0, e1)
    launches = dev.launch_count() - l0
    cuda_sync(dev)
    ranks.barrier()
    ms_total = ranks.max_f32(ms_total)
    # the dominant kernel alone (GEMM + fused epilogue), events around each launch
    evs = [(dev.event(), dev.event()) for _ in range(args.steps)]
    for i in range(args.steps):
        s = i % NSETS
        dev.quant_rows_i8(dA[s], M, K, dQa[s], dSa[s])
        dev.record(evs[i][0])
        dev.linear_i8_fwd(dQa[s], dSa[s], dQw[s], dSw[s], db, dY[s], M, N, K, True)
        dev.record(evs[i][1])
    dev.sync()
    gemm_ms = statistics.mean(dev.elapsed_ms(a, c) for a, c in evs)
    if M < 1024:
        # a launch of a few microseconds is shorter than what an event pair around it adds: time
        # the GEMM launches as one batch instead (operands still rotating), one event pair around it
        dev.record(e0)
        for i in range(args.steps):
            s = i % NSETS
            dev.linear_i8_fwd(dQa[s], dSa[s], dQw[s], dSw[s], db, dY[s], M, N, K, True)
        dev.record(e1)
        gemm_ms = dev.elapsed_ms(e0, e1) / args.steps
    assert dev.check_status() == 0

    # end to end through the C ABI with host buffers (pinned), copies inside the timed region: every
    # step's A comes from the host and every step's Y goes back; the copy of the next A and of the
    # last Y run on the library's copy streams while the current step computes (double buffering)
    import ctypes as C
    hA, hY = [C.c_void_p(), C.c_void_p()], [C.c_void_p(), C.c_void_p()]
    for h in hA:
        assert dev.lib.vtlb_host_alloc(A.nbytes, C.byref(h)) == 0
        C.memmove(h.value, A.ctypes.data, A.nbytes)
    for h in hY:
        assert dev.lib.vtlb_host_alloc(M * N * 4, C.byref(h)) == 0

    def e2e_run(steps):
        dev.copy_h2d_async(dA[0], hA[0].value, A.nbytes)
        for i in range(steps):
            s = i % NSETS
            dev.copy_wait(dev.COPY_IN_BEFORE_COMPUTE)          # A of this step has landed
            if i + 1 < steps:                                  # next A into a buffer no step is using
                dev.copy_h2d_async(dA[(i + 1) % NSETS], hA[(i + 1) % 2].value, A.nbytes)
            dev.quant_rows_i8(dA[s], M, K, dQa[s], dSa[s])
            dev.linear_i8_fwd(dQa[s], dSa[s], dQw[s], dSw[s], db, dY[s], M, N, K, True)
            dev.copy_wait(dev.COPY_OUT_BEFORE_COMPUTE)         # later steps wait for the earlier copies out
            dev.copy_d2h_async(hY[i % 2].value, dY[s], M * N * 4)
        dev.copy_wait(dev.COPY_OUT_DONE)                       # the last result is on the host

    e2e_run(3)
    cuda_sync(dev)
    ranks.barrier()
    t0 = time.perf_counter()
    e2e_run(args.steps)
    cuda_sync(dev)
    e2e_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = ranks.max_f32(e2e_ms)
    clocks = sampler.stop() if ranks.rank == 0 else None
    for h in hA + hY:
        dev.lib.vtlb_host_free(h)

    ops_step = 2.0 * M * N * K * ranks.world
    ms_step = ms_total / args.steps
    pk = peaks()
    int8_peak = 2.0 * pk["bf16_tflops"]  # INT8 issues at twice the bf16 rate on B200
    gemm_tops = 2.0 * M * N * K / (gemm_ms * 1e-3) / 1e12
    # roofline of the dominant kernel (the GEMM with its fused epilogue).  It is bound by the tensor
    # cores once 2*M*N*K / peak exceeds the time HBM needs for the operands (M >= 256 at N = K = 4096);
    # with fewer rows it is bound by streaming the weight codes once.
    op_bytes = float(N * K + M * K + 4 * M * N + 4 * (M + 2 * N))
    tensor_bound = 2.0 * M * N * K / (int8_peak * 1e12) >= op_bytes / (pk["hbm_gbs"] * 1e9)
    if M <= 2:
        kname = "gemv_i8_kernel (dp4a, one output channel per warp, a whole weight row in flight)"
    elif M <= 128:
        kname = ("skinny::gemm_i8_skinny_kernel (tcgen05 kind::i8 with the weights on the M side, K cut "
                 "across a cluster of 4 CTAs, partial sums added through distributed shared memory)")
    elif M < 1024:
        kname = "gemm::gemm_tc_kernel<KIND_I8, EpiDequant> (tcgen05 kind::i8, one CTA per tile, TMA-store epilogue)"
    else:
        kname = ("gemm2::gemm_pair_kernel<KIND_I8, EpiDequant> (tcgen05 kind::i8, cta_group::2, "
                 "fused dequant+bias+ReLU, TMA-store epilogue, K-split of surplus tiles)")
    if tensor_bound:
        roof = {"bound": "tensor", "kernel": kname, "achieved": gemm_tops, "peak": int8_peak, "unit": "TFLOP/s",
                "frac": gemm_tops / int8_peak,
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel on the
                # M = 4096 workload, from the ncu capture summarised in
                # profiles/gemm_i8_pair_fused_4096.md (algorithmic operand bytes: 33.6 MB read)
                "traffic": 59.9e6 if M == I8_M else None,
                "traffic_unit": "bytes per launch (ncu, 34.55 MB read + 25.38 MB written)" if M == I8_M else None,
                "algorithmic_ops_per_launch": 2.0 * M * N * K,
                "peak_source": f"2 x bf16_tflops of {pk['_source']} (cuBLAS bf16 burst rate; "
                               "dense INT8 issues at twice the bf16 rate)",
                "kernel_ms": gemm_ms}
    else:
        gbs = op_bytes / (gemm_ms * 1e-3) / 1e9
        # ncu on the M = 16 launch (profiles/gemm_i8_skinny_m16.md): 16.9 MB of DRAM traffic against 17.1 MB
        # of algorithmic bytes -- every weight code read once; other row counts scaled by their bytes
        roof = {"bound": "hbm", "kernel": kname, "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": gbs / pk["hbm_gbs"], "traffic": op_bytes * (16.9 / 17.14),
                "traffic_unit": "bytes per launch (ncu capture at M = 16, scaled by the algorithmic bytes)",
                "algorithmic_bytes_per_launch": op_bytes,
                "peak_source": f"hbm_gbs of {pk['_source']}", "kernel_ms": gemm_ms}
    out = None
    if ranks.rank == 0:
        cpu_tops, cores, sample, _, _ = cpu_int8_sample(A, W, b) if ranks.world == 1 else (None, None, None, None, None)
        out = {
            "metric": "int8_quantized_linear_fwd_tops", "value": ops_step / (ms_step * 1e-3) / 1e12,
            "unit": "TOPS", "n_gpus": ranks.world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
            "config": {"workload": "INT8 quantised Linear forward (baseline config 2"
                       + ("" if M == I8_M else f", M = {M} of its M sweep") + "): per-row "
                       f"dynamic quantisation of A f32 [{M},4096] ~N(0,1) + int8 GEMM against "
                       "pre-quantised W [4096,4096] ~N(0,0.02) + fused dequant+bias+ReLU",
                       "M": M, "N_per_gpu": N, "K": K, "parallelism":
                       f"output-column sharded x{ranks.world}, activations replicated, no collective",
                       "l2": f"every operand rotates over {NSETS} copies ({NSETS * set_bytes / 2**20:.0f} MiB) "
                             "between steps, larger than the 126 MB L2"},
            "e2e": {"value": ops_step / (e2e_ms / args.steps * 1e-3) / 1e12, "unit": "TOPS",
                    "h2d_bytes_per_step": int(A.nbytes), "d2h_bytes_per_step": int(M * N * 4),
                    "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": roof,
        }
        if cpu_tops is not None:
            out["cpu_baseline"] = {"value": cpu_tops, "unit": "TOPS", "cores": cores, "kind": "port",
                                   "sample": sample}
    ranks.close()
    dev.close()
    return out


def run_int8_reference(args, ranks):
    """The CPU arm: the oracle's quantised linear forward on all host threads, each step a
    bounded sample (a block of rows of A against the full weight matrix)."""
    if ranks.rank != 0:
        ranks.close()
        return None
    A, W, b = make_int8_inputs(2, 0)
    from oracle import oracle
    oracle.build()
    wq, sw = oracle.quant_rows_i8(W)
    # rows per step sized so that the whole --steps/--warmup run stays near a minute
    _, cores, _, rows, dt = cpu_int8_sample(A, W, b, budget_s=min(20.0, max(0.02, 60.0 / max(1, args.steps + args.warmup))))
    for _ in range(args.warmup):
        oracle.linear_i8_fwd(A[:rows], wq, sw, b, True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.linear_i8_fwd(A[:rows], wq, sw, b, True)
    ms_step = (time.perf_counter() - t0) * 1e3 / args.steps
    tops = 2.0 * rows * I8_N * I8_K / (ms_step * 1e-3) / 1e12
    sample = f"each step = first {rows} of {I8_M} rows of A against all {I8_N} channels"
    out = {"impl": "reference", "metric": "int8_quantized_linear_fwd_tops", "value": tops,
           "unit": "TOPS", "n_gpus": ranks.world, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
           "config": {"workload": "INT8 quantised Linear forward (baseline config 2), CPU oracle", "M": rows,
                      "N_per_gpu": I8_N, "K": I8_K},
           "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port", "sample": sample},
           "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    ranks.close()
    return out


def use_all_host_threads():
    """The CPU arm runs on every host core.  torch.distributed.run exports OMP_NUM_THREADS=1 to its
    workers, which would leave the oracle's OpenMP loops and NumPy's BLAS on one thread at N > 1."""
    n = os.cpu_count() or 1
    try:
        from oracle import oracle
        oracle.build()
        oracle.set_threads(n)
    except Exception as e:  # an oracle built before the setter existed: report, keep going
        print(f"bench: could not raise the oracle's thread count: {e}", file=sys.stderr)
    try:
        import threadpoolctl
        threadpoolctl.threadpool_limits(limits=n)
    except Exception as e:
        print(f"bench: could not raise the BLAS thread count: {e}", file=sys.stderr)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="int8_linear")
    ap.add_argument("--rows", type=int, default=None,
                    help="int8_linear: rows M of the activations (the M sweep of baseline config 2; "
                         "default 4096); training workloads: global batch override, for small "
                         "profiling captures")
    args = ap.parse_args()
    defaults = {"int8_linear": (2000, 20), "mlp_c1": (1000, 20), "mlp_c4": (20, 3), "cnn_c3": (50, 5),
                "int8_mlp_c5": (20, 3), "ckpt_c4": (20, 3)}
    if args.workload not in defaults:
        raise SystemExit(f"unknown workload {args.workload}; choose from {sorted(defaults)}")
    if args.steps is None:
        args.steps = defaults[args.workload][0] if args.impl == "ours" else 3
    if args.warmup is None:
        args.warmup = defaults[args.workload][1] if args.impl == "ours" else 1
    if args.impl == "ours":
        args.warmup = max(args.warmup, 3)
    ranks = Ranks(args.gpus)
    if args.impl == "reference" and ranks.rank == 0:
        use_all_host_threads()
    if args.workload == "int8_linear":
        out = run_int8_reference(args, ranks) if args.impl == "reference" else run_int8(args, ranks)
    elif args.workload == "int8_mlp_c5":
        import bench_infer
        if args.impl == "reference":
            out = bench_infer.run_reference(args, ranks)
        else:
            out = bench_infer.run(args, ranks, ClockSampler, peaks, cuda_sync)
    elif args.workload == "ckpt_c4":
        import bench_ckpt
        if args.impl == "reference":
            out = bench_ckpt.run_reference(args, ranks)
        else:
            out = bench_ckpt.run(args, ranks, ClockSampler, peaks, cuda_sync)
    else:
        import bench_train
        if args.impl == "reference":
            out = bench_train.run_reference(args, ranks)
        else:
            out = bench_train.run(args, ranks, ClockSampler, peaks, cuda_sync)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
