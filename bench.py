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

    def snapshot(self):
        """Summary of the samples taken since the last snapshot (or since start)."""
        mark = getattr(self, "_mark", 0)
        part = self.samples[mark:]
        self._mark = len(self.samples)
        return self._summary(part)

    def stop(self):
        self.stop_flag = True
        if self.thread:
            self.thread.join(timeout=2)
        return self._summary(self.samples)

    def _summary(self, samples):
        if not samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "samples": 0, "reasons": [self.err or "no samples"]}
        nv = self.nv
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        reasons = sorted(k for k, bit in names.items() if any(s[1] & bit for s in samples))
        # clocks idle low between kernels: the figure that matters is the clock under load
        top = sorted(s[0] for s in samples)
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
            self._red = dev.zeros(64, np.float32)

    def barrier(self):
        if self.dist:
            self.dist.barrier()

    def max_f32(self, x: float) -> float:
        return self.max_many([x])[0]

    def max_many(self, xs):
        """Element-wise maximum over the ranks of up to 64 numbers (the library's own NCCL
        communicator carries it)."""
        xs = [float(x) for x in xs]
        if self.world == 1:
            return xs
        assert len(xs) <= 64
        dev = self.dev
        h = np.zeros(64, np.float32)
        h[:len(xs)] = xs
        dev.h2d_raw(self._red, h.ctypes.data, 256)
        dev.sync()
        dev.allreduce_max_f32_async(self._red, 64)
        dev.comm_wait()
        return [float(v) for v in self._red.numpy()[:len(xs)]]

    def gather_objects(self, obj):
        """[obj of rank 0, ..., obj of rank N-1] on every rank (control plane, gloo)."""
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj)
        return out

    def close(self):
        if self.dist:
            self.dist.barrier()
            self.dist.destroy_process_group()


def timed_repeats(dev, ranks, run_steps, steps, min_repeat_s=0.25, min_repeats=5, max_total_s=8.0):
    """Times `run_steps(n)` (n steps enqueued on the compute stream) as several repeats, each
    bracketed by a rank barrier and a device synchronisation on both sides and by one CUDA event
    pair on the launching stream.  A repeat runs a whole multiple of `steps` steps, as many as it
    takes to keep the device busy for `min_repeat_s`; at least `min_repeats` repeats are taken
    (fewer only if they would exceed `max_total_s`).  Returns (ms per step of every repeat, maximum
    over the ranks; steps per repeat)."""
    e0, e1 = dev.event(), dev.event()

    def one(n):
        dev.sync()
        ranks.barrier()
        dev.record(e0)
        run_steps(n)
        dev.record(e1)
        ms = dev.elapsed_ms(e0, e1)
        dev.sync()
        ranks.barrier()
        return ms

    probe = ranks.max_f32(one(steps))  # also the last warm-up: clocks are up, caches in their steady state
    mult = max(1, int(np.ceil(min_repeat_s * 1e3 / max(probe, 1e-3))))
    per_repeat_s = probe * mult * 1e-3
    reps = max(min_repeats, 1)
    if reps * per_repeat_s > max_total_s:
        reps = max(2, int(max_total_s / per_repeat_s))
    n = steps * mult
    local = [one(n) / n for _ in range(reps)]
    out = []
    for i in range(0, len(local), 64):
        out += ranks.max_many(local[i:i + 64])
    return out, n


def spread(ms_list):
    """median / min / max of the per-step times of the repeats."""
    return {"repeats": len(ms_list), "median_ms_per_step": statistics.median(ms_list),
            "min_ms_per_step": min(ms_list), "max_ms_per_step": max(ms_list)}


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


class Int8Case:
    """Operands of one point of config 2 (M rows of activations against this rank's 4096 x 4096
    weight shard), every operand in as many rotating copies as it takes to exceed the 126 MB L2."""

    def __init__(self, dev, M, rank, A=None, Wb=None):
        self.dev, self.M, self.N, self.K = dev, M, I8_N, I8_K
        M, N, K = self.M, self.N, self.K
        if A is None:
            A, W, b = make_int8_inputs(2, rank, M)
        else:
            W, b = Wb
        self.A, self.W, self.b = A, W, b
        self.set_bytes = M * K * 5 + M * N * 4 + N * K
        self.nsets = n = max(4, -(-170_000_000 // self.set_bytes))
        self.dA = [dev.to_device(A) for _ in range(n)]
        self.dQa = [dev.zeros((M, K), np.int8) for _ in range(n)]
        self.dSa = [dev.zeros(M) for _ in range(n)]
        self.dY = [dev.zeros((M, N)) for _ in range(n)]
        dW = dev.to_device(W)
        self.dQw = [dev.zeros((N, K), np.int8) for _ in range(n)]
        self.dSw = [dev.zeros(N) for _ in range(n)]
        self.db = dev.to_device(b)
        for i in range(n):  # weights are quantised once, ahead of time
            dev.quant_rows_i8(dW, N, K, self.dQw[i], self.dSw[i])
        dev.sync()
        dW.free()

    def quant(self, i):
        s = i % self.nsets
        self.dev.quant_rows_i8(self.dA[s], self.M, self.K, self.dQa[s], self.dSa[s])

    def gemm(self, i):
        s = i % self.nsets
        self.dev.linear_i8_fwd(self.dQa[s], self.dSa[s], self.dQw[s], self.dSw[s], self.db, self.dY[s],
                               self.M, self.N, self.K, True)

    def step(self, i):
        self.quant(i)
        self.gemm(i)

    def free(self):
        for b in self.dA + self.dQa + self.dSa + self.dY + self.dQw + self.dSw + [self.db]:
            b.free()

    # ---- the dominant kernel alone
    def gemm_kernel_ms(self, launches):
        """Average duration of the GEMM launch (fused epilogue included), operands rotating.  From
        M = 1024 on: one CUDA event pair around each launch.  Below, a launch of a few microseconds is
        shorter than what an event pair around it adds, so the launches are timed back to back as
        one batch behind their quantise passes."""
        dev = self.dev
        for i in range(self.nsets):
            self.quant(i)
        if self.M >= 1024:
            evs = [(dev.event(), dev.event()) for _ in range(launches)]
            for i in range(launches):
                self.quant(i)
                dev.record(evs[i][0])
                self.gemm(i)
                dev.record(evs[i][1])
            dev.sync()
            return statistics.mean(dev.elapsed_ms(a, c) for a, c in evs)
        e0, e1 = dev.event(), dev.event()
        for i in range(3):
            self.gemm(i)
        dev.record(e0)
        for i in range(launches):
            self.gemm(i)
        dev.record(e1)
        return dev.elapsed_ms(e0, e1) / launches

    def kernel_name(self):
        M = self.M
        if M <= 2:
            return "gemv_i8_kernel (dp4a, one output channel per warp, a whole weight row in flight)"
        if M <= 128:
            return ("skinny::gemm_i8_skinny_kernel (tcgen05 kind::i8 with the weights on the M side, K cut "
                    "across a cluster of 4 CTAs, partial sums added through distributed shared memory)")
        if M < 1024:
            return "gemm::gemm_tc_kernel<KIND_I8, EpiDequant> (tcgen05 kind::i8, one CTA per tile, TMA-store epilogue)"
        return ("gemm2::gemm_pair_kernel<KIND_I8, EpiDequant> (tcgen05 kind::i8, cta_group::2, "
                "fused dequant+bias+ReLU, TMA-store epilogue, K-split of surplus tiles)")

    def roofline(self, gemm_ms, pk):
        """Roofline object of the GEMM launch.  Bound by the tensor cores once 2*M*N*K / peak exceeds
        the time HBM needs for the operands (M >= 256 at N = K = 4096); with fewer rows by streaming
        the weight codes once."""
        M, N, K = self.M, self.N, self.K
        int8_peak = 2.0 * pk["bf16_tflops"]  # INT8 issues at twice the bf16 rate on B200
        op_bytes = float(N * K + M * K + 4 * M * N + 4 * (M + 2 * N))
        ops = 2.0 * M * N * K
        if ops / (int8_peak * 1e12) >= op_bytes / (pk["hbm_gbs"] * 1e9):
            tops = ops / (gemm_ms * 1e-3) / 1e12
            roof = {"bound": "tensor", "kernel": self.kernel_name(), "achieved": tops, "peak": int8_peak,
                    "unit": "TFLOP/s", "frac": tops / int8_peak, "traffic": None,
                    "algorithmic_ops_per_launch": ops,
                    "peak_source": f"2 x bf16_tflops of {pk['_source']} (cuBLAS bf16 burst rate; "
                                   "dense INT8 issues at twice the bf16 rate)",
                    "kernel_ms": gemm_ms}
            if M == I8_M:
                roof.update(NCU_TRAFFIC["pair_4096"])
        else:
            gbs = op_bytes / (gemm_ms * 1e-3) / 1e9
            t = NCU_TRAFFIC["skinny_m16"]
            roof = {"bound": "hbm", "kernel": self.kernel_name(), "achieved": gbs, "peak": pk["hbm_gbs"],
                    "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                    "traffic": op_bytes * t["traffic_per_algorithmic_byte"], "traffic_source": t["traffic_source"],
                    "algorithmic_bytes_per_launch": op_bytes,
                    "peak_source": f"hbm_gbs of {pk['_source']}", "kernel_ms": gemm_ms}
        return roof


# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) is not measurable inside a
# timed run; these are the figures of the ncu captures of the same launches, and say so.
NCU_TRAFFIC = {
    "pair_4096": {"traffic": 59.9e6,
                  "traffic_source": "ncu capture of one launch at M = N = K = 4096 (34.55 MB read + 25.38 MB "
                                    "written; most of the 67 MB output is still in L2 when the kernel ends), "
                                    "not measured in this run"},
    "skinny_m16": {"traffic_per_algorithmic_byte": 16.9 / 17.14,
                   "traffic_source": "ncu capture of one launch at M = 16 (16.9 MB of DRAM traffic against "
                                     "17.14 MB of algorithmic bytes), scaled by the algorithmic bytes; not "
                                     "measured in this run"},
}


def run_int8(args, ranks):
    from vtl_b200 import capi
    dev = capi.Device(ranks.local_rank)
    ranks.attach(dev)
    M, N, K = (args.rows or I8_M), I8_N, I8_K
    case = Int8Case(dev, M, ranks.rank)
    A, W, b = case.A, case.W, case.b
    NSETS, set_bytes = case.nsets, case.set_bytes
    dA, dY = case.dA, case.dY

    cuda_sync(dev)  # also pays the one-off import costs now, not between warm-up and timing
    sampler = ClockSampler(ranks.local_rank)
    if ranks.rank == 0:
        sampler.start()  # keeps sampling through all timed passes below
    ranks.barrier()
    for i in range(args.warmup):  # directly before the timed region: the GPU must not idle
        case.step(i)              # (and drop its clocks) between warm-up and timing
    dev.sync()
    # the dominant kernel alone (GEMM + fused epilogue), straight after the warm-up: a few
    # milliseconds of launches, timed in isolation (the burst regime of the clocks)
    gemm_ms = case.gemm_kernel_ms(min(max(args.steps, 20), 200))
    kernel_clocks = sampler.snapshot() if ranks.rank == 0 else None
    # what the tensor cores do with INT8 MMAs when nothing has to be loaded (same clocks regime)
    yard_burst = dev.int8_issue_yardstick(20000)
    # whole steps: repeats of K-step regions, each behind a barrier + sync, one event pair per region;
    # seconds of back-to-back steps, so these run under the power cap
    l0 = dev.launch_count()
    per_step, steps_per_repeat = timed_repeats(dev, ranks, lambda n: [case.step(i) for i in range(n)], args.steps)
    launches = dev.launch_count() - l0
    ms_step = statistics.median(per_step)
    step_clocks = sampler.snapshot() if ranks.rank == 0 else None
    yard_loaded = dev.int8_issue_yardstick(20000)  # again, straight after seconds of load (power-capped clocks)
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
            case.step(i)
            dev.copy_wait(dev.COPY_OUT_BEFORE_COMPUTE)         # later steps wait for the earlier copies out
            dev.copy_d2h_async(hY[i % 2].value, dY[s], M * N * 4)
        dev.copy_wait(dev.COPY_OUT_DONE)                       # the last result is on the host

    def e2e_timed(steps):
        cuda_sync(dev)
        ranks.barrier()
        t0 = time.perf_counter()
        e2e_run(steps)
        cuda_sync(dev)
        return (time.perf_counter() - t0) * 1e3

    e2e_run(3)
    probe = ranks.max_f32(e2e_timed(args.steps))
    mult = max(1, int(np.ceil(250.0 / max(probe, 1e-3))))
    e2e_steps = args.steps * mult
    e2e_per_step = ranks.max_many([e2e_timed(e2e_steps) / e2e_steps for _ in range(5)])
    e2e_ms_step = statistics.median(e2e_per_step)
    for h in hA + hY:
        dev.lib.vtlb_host_free(h)

    pk = peaks()
    roof = case.roofline(gemm_ms, pk)
    # the M sweep of config 2: the GEMM launch alone at every row count (single-GPU runs only)
    sweep = None
    if ranks.world == 1 and not args.rows:
        sweep = []
        case.free()
        for m in (1, 16, 128, 1024, 8192):
            c = Int8Case(dev, m, ranks.rank, A=A[:m] if m <= M else None, Wb=(W, b) if m <= M else None)
            for i in range(5):
                c.step(i)
            k_ms = c.gemm_kernel_ms(200 if m < 1024 else 40)
            st, _ = timed_repeats(dev, ranks, lambda n, c=c: [c.step(i) for i in range(n)], 50, min_repeat_s=0.05,
                                  min_repeats=3, max_total_s=1.0)
            r = c.roofline(k_ms, pk)
            sweep.append({"M": m, "kernel_ms": k_ms, "bound": r["bound"], "achieved": r["achieved"],
                          "unit": r["unit"], "frac": r["frac"], "step_ms": statistics.median(st),
                          "kernel": r["kernel"].split(" (")[0]})
            c.free()
        assert dev.check_status() == 0
    clocks = sampler.stop() if ranks.rank == 0 else None

    ops_step = 2.0 * M * N * K * ranks.world
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
            "timing": dict(spread(per_step), steps_per_repeat=steps_per_repeat,
                           note="value and ms_per_step are the median repeat; every repeat is a whole multiple of "
                                "--steps steps behind a barrier and a device synchronisation, timed by one CUDA "
                                "event pair, maximum over the ranks"),
            "e2e": {"value": ops_step / (e2e_ms_step * 1e-3) / 1e12, "unit": "TOPS",
                    "h2d_bytes_per_step": int(A.nbytes), "d2h_bytes_per_step": int(M * N * 4),
                    "ms_per_step": e2e_ms_step, "repeats": len(e2e_per_step),
                    "min_ms_per_step": min(e2e_per_step), "max_ms_per_step": max(e2e_per_step),
                    "steps_per_repeat": e2e_steps},
            "gpu_launches": int(launches),
            "clocks": dict(step_clocks, whole_run=clocks,
                           note="sampled through NVML during the timed repeats of whole steps; whole_run covers "
                                "every pass of this process (kernel-alone pass, repeats, end-to-end, sweep)"),
            "roofline": dict(roof, clocks=kernel_clocks,
                             int8_issue_yardstick={
                                 "tops_after_warmup": yard_burst, "tops_after_sustained_load": yard_loaded,
                                 "frac_of_yardstick": (roof["achieved"] / yard_burst) if roof["bound"] == "tensor" else None,
                                 "what": "this library's own kernel issuing tcgen05.mma.kind::i8 (cta_group::2, 256x256x32) "
                                         "back to back on operands resident in shared memory, no loads: the INT8 "
                                         "ceiling measured on this GPU, beside the 2 x bf16 proxy used as peak"}),
        }
        if sweep is not None:
            out["sweep"] = sweep
        if cpu_tops is not None:
            out["cpu_baseline"] = {"value": cpu_tops, "unit": "TOPS", "cores": cores, "kind": "port",
                                   "sample": sample}
    dev.close()
    return out


def run_int8_reference(args, ranks):
    """The CPU arm: the oracle's quantised linear forward on all host threads.  A step is the whole
    configuration (all 4096 rows of A against the full weight matrix, about 1.7 s on 16 cores); only
    if --steps + --warmup of those would run past four minutes is a step cut to the first rows of A,
    and the line then says so in config.M."""
    if ranks.rank != 0:
        return None
    A, W, b = make_int8_inputs(2, 0)
    from oracle import oracle
    oracle.build()
    wq, sw = oracle.quant_rows_i8(W)
    t0 = time.perf_counter()
    oracle.linear_i8_fwd(A[:256], wq, sw, b, True)
    oracle.linear_i8_fwd(A[:256], wq, sw, b, True)
    t_full = (time.perf_counter() - t0) / 2 * (I8_M / 256)
    rows = I8_M
    total = (args.steps + args.warmup) * t_full
    if total > 240.0:
        rows = max(32, int(I8_M * 240.0 / total) // 32 * 32)
    cores = oracle.max_threads()
    for _ in range(args.warmup):
        oracle.linear_i8_fwd(A[:rows], wq, sw, b, True)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.linear_i8_fwd(A[:rows], wq, sw, b, True)
    ms_step = (time.perf_counter() - t0) * 1e3 / args.steps
    tops = 2.0 * rows * I8_N * I8_K / (ms_step * 1e-3) / 1e12
    sample = (f"each step = all {I8_M} rows of A against all {I8_N} channels (the whole configuration)" if rows == I8_M
              else f"each step = first {rows} of {I8_M} rows of A against all {I8_N} channels")
    out = {"impl": "reference", "metric": "int8_quantized_linear_fwd_tops", "value": tops,
           "unit": "TOPS", "n_gpus": ranks.world, "steps": args.steps, "warmup": args.warmup,
           "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
           "config": {"workload": "INT8 quantised Linear forward (baseline config 2), CPU oracle", "M": rows,
                      "N_per_gpu": I8_N, "K": I8_K},
           "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": cores, "kind": "port", "sample": sample},
           "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
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
    ap.add_argument("--headline-only", action="store_true",
                    help="default workload: skip the dp_train / tp_infer objects (configs 4 and 5) and time "
                         "config 2 alone, e.g. for profiler captures")
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
    # stdout carries exactly one JSON line: libraries that print to file descriptor 1 (NCCL prints its
    # version there) are sent to stderr for the length of the run, the line goes to the real stdout
    sys.stdout.flush()
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    ranks = Ranks(args.gpus)
    if args.impl == "reference" and ranks.rank == 0:
        use_all_host_threads()
    if args.workload == "int8_linear":
        out = run_int8_reference(args, ranks) if args.impl == "reference" else run_int8(args, ranks)
        if args.impl == "ours" and not args.rows and not args.headline_only:
            # the two workloads that carry collectives, in the same process and on the same ranks:
            # config 4 (data-parallel f32 training, gradient all-reduce) and config 5 (column-sharded
            # INT8 inference, all-gather of activations), each with its parity checks
            import bench_infer
            import bench_train
            me = sys.modules[__name__]
            extra = {}
            for key, fn in (("dp_train", bench_train.run_dp), ("tp_infer", bench_infer.run_tp)):
                try:
                    extra[key] = fn(ranks, me)
                except Exception as e:  # the headline above stands; the failure is reported in its place
                    extra[key] = {"error": f"{type(e).__name__}: {e}"}
                    print(f"bench: {key} failed on rank {ranks.rank}: {e}", file=sys.stderr)
            if out is not None:
                out.update(extra)
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
    ranks.close()
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
