"""INT8 weight-quantised MLP inference workload of bench.py (`--workload int8_mlp_c5`),
baseline config 5: 4 layers 8192 -> 28672 -> 8192 -> 28672 -> 8192, weights ~N(0,0.02)
quantised per output channel, activations quantised per row on the fly, a batch of 16384
tokens ~N(0,1), ReLU between layers.

With N ranks every layer is sharded by output columns (rank r owns N_l/N channels and their
scales) and the activations are exchanged between layers:
    local f32 slab [M, N_l/N]  ->  row max-abs  ->  NCCL all-reduce(max) over ranks
    ->  quantise the slab with the global row scale  ->  all-gather of the int8 codes (each rank
        copies its codes into the peers' buffers with the copy engines; NCCL's kernel on request)
The next layer's GEMM reads the gathered shards in place (vtlb_linear_i8_fwd_sharded_a).
The last layer's output stays sharded.  Strong scaling: the total work is fixed."""
from __future__ import annotations

import ctypes as C
import os
import statistics
import sys
import time

import numpy as np

DIMS = [8192, 28672, 8192, 28672, 8192]
TOKENS = 16384


def total_ops(tokens=TOKENS):
    return sum(2.0 * tokens * DIMS[i] * DIMS[i + 1] for i in range(len(DIMS) - 1))


class ShardedInt8MLP:
    """One rank's part of the model and its activation buffers.

    With more than one rank the tokens are processed as `chunks` independent row blocks (rows
    are quantised independently, so a block can run ahead through the layers): while the codes
    of one block are all-gathered on the communication stream, the GEMM of the next block runs
    on the compute stream.

    `exchange` (obj -> [obj of every rank], a host channel) switches the all-gathers from NCCL's
    kernel to the copy engines: each rank exports its receive buffers to the others, and a
    gather is every rank copying its codes straight into the peers' buffers, so the SMs stay
    with the GEMMs (VTLB_C5_GATHER=nccl keeps NCCL's all-gather)."""

    def __init__(self, dev, world, rank, tokens=TOKENS, dims=DIMS, seed=5, chunks=None, exchange=None):
        self.dev, self.R, self.rank, self.M, self.dims = dev, world, rank, tokens, dims
        self.push = bool(world > 1 and exchange is not None
                         and os.environ.get("VTLB_C5_GATHER", "push") != "nccl")
        self._shared, self._opened = [], []
        self.C = chunks if chunks else (int(os.environ.get("VTLB_C5_ROW_BLOCKS", "2")) if world > 1 else 1)
        assert tokens % self.C == 0
        self.Mc = tokens // self.C
        self.layers = []
        for li in range(len(dims) - 1):
            K, N = dims[li], dims[li + 1]
            n = N // world
            # the rank's rows of W: generated shard by shard so no rank ever holds the full matrix
            rng = np.random.default_rng([seed, li, rank])
            W = rng.standard_normal((n, K), dtype=np.float32) * np.float32(0.02)
            b = rng.standard_normal(n, dtype=np.float32) * np.float32(0.01)
            dW = dev.to_device(W)
            dQ, dS = dev.zeros((n, K), np.int8), dev.zeros(n)
            dev.quant_rows_i8(dW, n, K, dQ, dS)
            dev.sync()
            dW.free()
            L = dict(K=K, N=N, n=n, Wq=dQ, sw=dS, bias=dev.to_device(b),
                     Y=dev.zeros((tokens, n)), amax=dev.zeros(tokens), sa=dev.zeros(tokens))
            self.layers.append(L)
        hidden = self.layers[:-1]  # the layers whose output is exchanged
        if self.push and not self._open_shared(hidden, exchange):
            self.push = False      # every rank took the same decision: NCCL's all-gather instead
            print("bench_infer: gather buffers could not be shared between the ranks' processes; "
                  "using NCCL's all-gather", file=sys.stderr)
        for L in self.layers:
            if "q_all_ptr" not in L:
                # per row block: the gathered shards [world][Mc][n]
                L["q_local"] = dev.zeros((tokens, L["n"]), np.int8)
                L["q_all"] = dev.zeros((self.C, world, self.Mc, L["n"]), np.int8)
                L["q_all_ptr"] = L["q_all"].ptr
        self.q_in, self.sa_in = dev.zeros((tokens, dims[0]), np.int8), dev.zeros(tokens)

    def _open_shared(self, hidden, exchange) -> bool:
        """Allocates this rank's gather buffers, ships their handles and opens the peers'.  After
        each of the two steps the ranks tell each other whether it worked, so that either all of
        them use the copy-engine route or none does; on failure everything is undone."""
        from vtl_b200.capi import VtlbError
        dev, R = self.dev, self.R
        inject = os.environ.get("VTLB_C5_FAIL_SHARING") == str(self.rank)  # failure made on the host, for tests
        ok = True
        try:
            if inject:
                raise VtlbError(-1, "injected")
            for L in hidden:
                ptr, handle = dev.shared_alloc(self.C * R * self.Mc * L["n"])
                self._shared.append(ptr)
                L["q_all_ptr"], L["handle"] = ptr, handle
        except VtlbError:
            ok = False
        if all(exchange(ok)):
            table = exchange([L["handle"] for L in hidden])
            try:
                for li, L in enumerate(hidden):
                    L["peers"] = []
                    for r in range(R):
                        L["peers"].append(None if r == self.rank else dev.shared_open(table[r][li]))
                        if L["peers"][-1]:
                            self._opened.append(L["peers"][-1])
            except VtlbError:
                ok = False
            if all(exchange(ok)):  # also: all handles are open before any rank can start pushing
                # row maxima are all-reduced beside the copies, not queued behind them
                if os.environ.get("VTLB_C5_SMALL_LANE", "1") != "0":
                    dev.comm_small_lane()
                return True
        for p in self._opened:
            dev.shared_close(p)
        exchange(0)  # nobody has a peer's buffer mapped any more (every rank gets here, with or without buffers)
        for p in self._shared:
            dev.shared_free(p)
        self._opened, self._shared = [], []
        for L in hidden:
            for k in ("q_all_ptr", "handle", "peers"):
                L.pop(k, None)
        return False

    def close(self, barrier=None):
        """Unmaps the peers' buffers, then frees this rank's.  Call it on every rank once no rank is
        still copying; `barrier` (a host barrier over the ranks) separates the two halves, because an
        exported buffer must not be freed while another process still has it mapped."""
        for p in self._opened:
            self.dev.shared_close(p)
        self._opened = []
        if barrier is not None and self._shared:
            barrier()
        for p in self._shared:
            self.dev.shared_free(p)
        self._shared = []

    def forward(self, dX, y_out=None):
        """`y_out`: an alternative buffer for the last layer's output (for double buffering)."""
        dev, M, R, C, Mc = self.dev, self.M, self.R, self.C, self.Mc
        dev.quant_rows_i8(dX, M, self.dims[0], self.q_in, self.sa_in)  # replicated input
        # per row block: where its quantised activations live and in how many column shards
        aq = [self.q_in.ptr + c * Mc * self.dims[0] for c in range(C)]
        sa = [self.sa_in.ptr + 4 * c * Mc for c in range(C)]
        shards = 1
        # Every wait is for one collective, not for the communication stream as a whole: mark c follows
        # the all-gather of row block c (bulk lane), mark 32 + c its max all-reduce (small lane).
        gathered = [False] * C       # an all-gather of the block is in flight
        for li, L in enumerate(self.layers):
            last = li + 1 == len(self.layers)
            n, K = L["n"], L["K"]
            for c in range(C):
                if gathered[c]:      # the block's codes must have arrived
                    dev.comm_wait_mark(c)
                    gathered[c] = False
                y = (y_out.ptr if (last and y_out is not None) else L["Y"].ptr) + 4 * c * Mc * n
                if last:
                    dev.linear_i8_fwd_sharded_a(aq[c], shards, sa[c], L["Wq"], L["sw"], L["bias"], y, Mc, n, K,
                                                relu=False)
                    continue
                amax = L["amax"].ptr + 4 * c * Mc
                sa_out = L["sa"].ptr + 4 * c * Mc
                q_all = L["q_all_ptr"] + c * R * Mc * n
                # the GEMM's epilogue also leaves the row maxima of its output slab (no second pass over Y)
                dev.linear_i8_fwd_amax(aq[c], shards, sa[c], L["Wq"], L["sw"], L["bias"], y, Mc, n, K, True, amax)
                if R > 1:
                    dev.allreduce_max_f32_async(amax, Mc)
                    dev.comm_mark(dev.LANE_SMALL, 32 + c)
                    dev.comm_wait_mark(32 + c)
                    if self.push:
                        # quantise into this rank's own part of the gathered block, then copy it
                        # into the same part of every peer's block
                        mine = (c * R + self.rank) * Mc * n
                        dev.quant_rows_i8(y, Mc, n, q_all + self.rank * Mc * n, sa_out, amax)
                        dev.allgather_push_async(q_all + self.rank * Mc * n,
                                                 [p + mine if p else None for p in L["peers"]], Mc * n)
                    else:
                        q_loc = L["q_local"].ptr + c * Mc * n
                        dev.quant_rows_i8(y, Mc, n, q_loc, sa_out, amax)
                        dev.allgather_async(q_loc, q_all, Mc * n)
                    dev.comm_mark(dev.LANE_BULK, c)
                    gathered[c] = True
                else:
                    dev.quant_rows_i8(y, Mc, n, q_all, sa_out, amax)
                aq[c], sa[c] = q_all, sa_out
            shards = R
        if R > 1:
            dev.comm_wait()  # nothing of this pass is left in flight (and the library forgets the operands it tracks)
        return y_out if y_out is not None else self.layers[-1]["Y"]


def cpu_sample(tokens=64, budget_s=15.0):
    """The oracle's unsharded forward on a few tokens, all host threads."""
    from oracle import oracle
    oracle.build()
    rng = np.random.default_rng(5)
    X = rng.standard_normal((tokens, DIMS[0]), dtype=np.float32)
    Ws = []
    for li in range(len(DIMS) - 1):
        W = rng.standard_normal((DIMS[li + 1], DIMS[li]), dtype=np.float32) * np.float32(0.02)
        Ws.append(oracle.quant_rows_i8(W) + ((rng.standard_normal(DIMS[li + 1]) * 0.01).astype(np.float32),))

    def fwd():
        A = X
        for i, (wq, sw, b) in enumerate(Ws):
            A = oracle.linear_i8_fwd(A, wq, sw, b, relu=(i + 1 < len(Ws)))
        return A

    fwd()
    n, t0 = 0, time.perf_counter()
    while n == 0 or time.perf_counter() - t0 < budget_s:
        fwd()
        n += 1
    dt = (time.perf_counter() - t0) / n
    return {"value": total_ops(tokens) / dt / 1e12, "unit": "TOPS", "cores": oracle.max_threads(), "kind": "port",
            "sample": f"{n} forward passes of {tokens} tokens (of {TOKENS}) through all four layers",
            "tokens_per_s": tokens / dt}, dt


def run_reference(args, ranks):
    if ranks.rank != 0:
        return None
    cb, dt = cpu_sample(budget_s=max(5.0, 20.0 * max(1, args.steps)))
    out = {"impl": "reference", "metric": "int8_mlp_inference_tops", "value": cb["value"], "unit": "TOPS",
           "n_gpus": ranks.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
           "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
           "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
           "config": {"workload": "INT8 MLP inference 8192-28672-8192-28672-8192 (baseline config 5), CPU oracle"},
           "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
           "e2e": {"value": cb["value"], "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    return out


def run(args, ranks, ClockSampler, peaks, cuda_sync):
    from vtl_b200 import capi
    dev = capi.Device(ranks.local_rank)
    ranks.attach(dev)
    model = ShardedInt8MLP(dev, ranks.world, ranks.rank, exchange=ranks.gather_objects)
    X = np.random.default_rng(5).standard_normal((TOKENS, DIMS[0]), dtype=np.float32)
    dX = dev.to_device(X)
    cuda_sync(dev)
    sampler = ClockSampler(ranks.local_rank)
    if ranks.rank == 0:
        sampler.start()
    ranks.barrier()
    for _ in range(args.warmup):
        model.forward(dX)
    dev.sync()
    ranks.barrier()
    l0 = dev.launch_count()
    e0, e1 = dev.event(), dev.event()
    dev.record(e0)
    for _ in range(args.steps):
        model.forward(dX)
    dev.record(e1)
    ms_total = dev.elapsed_ms(e0, e1)
    launches = dev.launch_count() - l0
    cuda_sync(dev)
    ranks.barrier()
    ms_total = ranks.max_f32(ms_total)
    # GEMM launches alone
    dev.profile_gemm(True)
    psteps = max(1, min(args.steps, 8))
    for _ in range(psteps):
        model.forward(dX)
    gemm_ms, gemm_n, gemm_ops = dev.profile_gemm_read()
    dev.profile_gemm(False)
    # end to end: tokens from pinned host memory in, this rank's slab of the output back
    last = model.layers[-1]
    hX, hY = C.c_void_p(), C.c_void_p()
    out_bytes = TOKENS * last["n"] * 4
    assert dev.lib.vtlb_host_alloc(X.nbytes, C.byref(hX)) == 0
    assert dev.lib.vtlb_host_alloc(out_bytes, C.byref(hY)) == 0
    C.memmove(hX.value, X.ctypes.data, X.nbytes)

    # tokens in from pinned host memory and the output slab back to it every step; the next input
    # and the last output are copied on the library's copy streams while the current pass computes
    dXs = [dX, dev.empty(X.shape, X.dtype)]
    last = model.layers[-1]
    dYs = [last["Y"], dev.empty(last["Y"].shape, np.float32)]

    def e2e_run(steps):
        dev.copy_h2d_async(dXs[0], hX.value, X.nbytes)
        for i in range(steps):
            dev.copy_wait(dev.COPY_IN_BEFORE_COMPUTE)
            if i + 1 < steps:
                dev.copy_h2d_async(dXs[(i + 1) % 2], hX.value, X.nbytes)
            y = model.forward(dXs[i % 2], y_out=dYs[i % 2])
            dev.copy_wait(dev.COPY_OUT_BEFORE_COMPUTE)
            dev.copy_d2h_async(hY.value, y, out_bytes)
        dev.copy_wait(dev.COPY_OUT_DONE)

    e2e_run(2)
    cuda_sync(dev)
    ranks.barrier()
    esteps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    e2e_run(esteps)
    cuda_sync(dev)
    e2e_ms = ranks.max_f32((time.perf_counter() - t0) * 1e3)
    clocks = sampler.stop() if ranks.rank == 0 else None
    assert dev.check_status() == 0
    out = None
    if ranks.rank == 0:
        pk = peaks()
        ms_step = ms_total / args.steps
        int8_peak = 2.0 * pk["bf16_tflops"]
        gemm_tops = gemm_ops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
        out = {"metric": "int8_mlp_inference_tops", "value": total_ops() / (ms_step * 1e-3) / 1e12, "unit": "TOPS",
               "n_gpus": ranks.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
               "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
               "dtype": "int8 x int8 -> int32, f32 scales", "data": "synthetic",
               "config": {"workload": "INT8 weight-quantised MLP inference, 4 layers 8192->28672->8192->28672->8192, "
                                      "16384 tokens ~N(0,1), per-row dynamic activation quantisation, ReLU between "
                                      "layers (baseline config 5)",
                          "tokens": TOKENS, "tokens_per_s": TOKENS / (ms_step * 1e-3),
                          "parallelism": (f"output columns sharded x{ranks.world}; per layer all-reduce(max) of row "
                                          "maxima (NCCL) and all-gather of int8 codes ("
                                          + ("copy engines into the peers' buffers" if model.push else "NCCL") + ")")
                          if ranks.world > 1 else "single GPU",
                          "l2": "weights (4 x 235 MB int8) and activations exceed the 126 MB L2"},
               "e2e": {"value": total_ops() / (e2e_ms / esteps * 1e-3) / 1e12, "unit": "TOPS",
                       "h2d_bytes_per_step": int(X.nbytes), "d2h_bytes_per_step": int(out_bytes),
                       "ms_per_step": e2e_ms / esteps},
               "gpu_launches": int(launches), "clocks": clocks,
               "roofline": {"bound": "tensor", "kernel": "INT8 GEMM launches of a forward pass (fused epilogue)",
                            "achieved": gemm_tops, "peak": int8_peak, "unit": "TFLOP/s",
                            "frac": gemm_tops / int8_peak if gemm_tops else None, "traffic": None,
                            "peak_source": f"2 x bf16_tflops of {pk['_source']}",
                            "kernel_ms_per_step": gemm_ms / psteps, "launches_per_step": gemm_n / psteps}}
        if ranks.world == 1:
            cb, _ = cpu_sample()
            out["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    dev.sync()
    ranks.barrier()  # no rank is still copying into a peer's buffer
    model.close(ranks.barrier)
    dev.close()
    return out


# ------------------------------------------------------------------ config 5 inside the default bench line
def sharded_parity(ranks, dev, dims=(1024, 4096, 1024, 4096, 1024), tokens=512, chunks=2):
    """The sharded forward on a reduced config 5 (same topology, widths / 8, 512 tokens), every
    rank's output slab collected on rank 0 and compared with the UNSHARDED CPU oracle: the int32
    GEMM is exact, max is associative and quantisation is element-wise, so the result must be the
    same bit for bit however many ranks share the columns.  Rank 0 returns the report."""
    model = ShardedInt8MLP(dev, ranks.world, ranks.rank, tokens=tokens, dims=list(dims), seed=55, chunks=chunks,
                           exchange=ranks.gather_objects)
    X = np.random.default_rng(56).standard_normal((tokens, dims[0]), dtype=np.float32)
    dX = dev.to_device(X)
    y = model.forward(dX)
    dev.sync()
    slabs = ranks.gather_objects(y.numpy())  # every rank is past its last copy into a peer's buffer
    model.close(ranks.barrier)
    if ranks.rank != 0:
        return None
    from oracle import oracle
    oracle.build()
    A = X
    for li in range(len(dims) - 1):
        Ws, bs = [], []
        for r in range(ranks.world):  # the shards as the ranks generated them
            rng = np.random.default_rng([55, li, r])
            n = dims[li + 1] // ranks.world
            Ws.append(rng.standard_normal((n, dims[li]), dtype=np.float32) * np.float32(0.02))
            bs.append(rng.standard_normal(n, dtype=np.float32) * np.float32(0.01))
        wq, sw = oracle.quant_rows_i8(np.concatenate(Ws))
        A = oracle.linear_i8_fwd(A, wq, sw, np.concatenate(bs), relu=(li + 2 < len(dims)))
    got = np.concatenate(slabs, axis=1)
    return {"config": f"{'-'.join(map(str, dims))}, {tokens} tokens, {chunks} row blocks, sharded x{ranks.world}, "
                      "against the unsharded CPU oracle",
            "bit_exact": bool(np.array_equal(got.view(np.uint32), A.view(np.uint32))),
            "max_abs_diff": float(np.abs(got - A).max())}


def run_tp(ranks, tools, steps=10, warmup=3):
    """Baseline config 5 on the ranks of this job (output columns sharded, strong scaling): TOPS, the
    GEMM launches alone, the exposed part of the per-layer exchange, and the parity check of the
    sharded pipeline.  Returns the object on rank 0."""
    from vtl_b200 import capi
    dev = capi.Device(ranks.local_rank)
    ranks.attach(dev)
    parity = sharded_parity(ranks, dev)
    model = ShardedInt8MLP(dev, ranks.world, ranks.rank, exchange=ranks.gather_objects)
    dX = dev.to_device(np.random.default_rng(5).standard_normal((TOKENS, DIMS[0]), dtype=np.float32))

    def run_steps(n):
        for _ in range(n):
            model.forward(dX)

    tools.cuda_sync(dev)
    ranks.barrier()
    run_steps(warmup)
    l0 = dev.launch_count()
    per_step, steps_per_repeat = tools.timed_repeats(dev, ranks, run_steps, steps, max_total_s=6.0)
    launches = dev.launch_count() - l0
    ms_step = statistics.median(per_step)
    psteps = 4
    dev.profile_gemm(True)
    run_steps(psteps)
    phases = dev.profile_read_phases()
    gemm_ms, gemm_n, gemm_ops = dev.profile_gemm_read()
    dev.profile_gemm(False)
    assert dev.check_status() == 0
    dev.sync()
    ranks.barrier()  # no rank is still copying into a peer's buffer
    push = model.push
    model.close(ranks.barrier)
    dev.close()
    if ranks.rank != 0:
        return None
    pk = tools.peaks()
    int8_peak = 2.0 * pk["bf16_tflops"]
    gemm_tops = gemm_ops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    return {"workload": "INT8 weight-quantised MLP inference, 4 layers 8192->28672->8192->28672->8192, 16384 tokens "
                        "~N(0,1), per-row dynamic activation quantisation, ReLU between layers (baseline config 5)",
            "metric": "int8_mlp_inference_tops", "value": total_ops() / (ms_step * 1e-3) / 1e12, "unit": "TOPS",
            "scaling": "strong", "tokens": TOKENS, "tokens_per_s": TOKENS / (ms_step * 1e-3), "ms_per_step": ms_step,
            "timing": dict(tools.spread(per_step), steps_per_repeat=steps_per_repeat),
            "gpu_launches": int(launches), "row_blocks": model.C,
            "gemm_ms_per_step": gemm_ms / psteps, "gemm_launches_per_step": gemm_n / psteps,
            "gemm_tops_per_gpu": gemm_tops, "gemm_frac_of_peak": gemm_tops / int8_peak if gemm_tops else None,
            "gemm_peak": int8_peak, "gemm_peak_source": f"2 x bf16_tflops of {pk['_source']}",
            "exchange_ms_per_step": {"quantise": phases["elementwise"][0] / psteps,
                                     "exposed_collective_wait": phases["comm_wait"][0] / psteps,
                                     "note": "quantise = the row-quantisation launches; exposed_collective_wait = "
                                             "time the compute stream stood idle until an all-reduce(max) or "
                                             "all-gather had finished (CUDA-event brackets, profiled passes)"},
            "parallelism": (f"output columns sharded x{ranks.world}; per layer and row block: all-reduce(max) of row "
                            "maxima (NCCL), quantise, all-gather of int8 codes ("
                            + ("copy engines into the peers' buffers" if push else "NCCL")
                            + "); the next GEMM reads the gathered "
                            "shards in place") if ranks.world > 1 else "single GPU",
            "parity": parity}
