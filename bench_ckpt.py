"""Checkpoint-payload workload of bench.py (`--workload ckpt_c4`): the parameters of baseline
config 4 (8 Linear layers of width 4096: 8 x (4096^2 + 4096) = 134.25 M f32 values) turned into the
text the reference's save_checkpoint stores (f64 big-endian bytes in base64,
nn/models/serialization.v:421-438) and back.

A step = encode every parameter tensor (16 launches).  The kernels are bound by HBM: 4 bytes read
and 32/3 bytes written per value.  Parameters are replicated in data-parallel training, so with N
ranks every rank encodes its own replica: replicas only, no collective."""
from __future__ import annotations

import ctypes as C
import os
import statistics
import time

import numpy as np

WIDTH, LAYERS = 4096, 8


def tensor_sizes():
    out = []
    for _ in range(LAYERS):
        out += [WIDTH * WIDTH, WIDTH]
    return out


def cpu_sample(budget_s=12.0):
    """The oracle's payload encoder (numpy widening + byte swap + base64) on one weight matrix."""
    from oracle import checkpoint as ock
    rng = np.random.default_rng(4)
    w = rng.standard_normal(WIDTH * WIDTH, dtype=np.float32)
    ock.encode_payload(w[:1024])
    reps, t0 = 0, time.perf_counter()
    while True:
        text = ock.encode_payload(w)
        reps += 1
        dt = time.perf_counter() - t0
        if dt > budget_s or reps >= 64:
            break
    bytes_ = (4 * w.size + len(text)) * reps
    return bytes_ / dt / 1e9, 1, f"{reps} encodings of one {WIDTH}x{WIDTH} weight matrix ({dt:.1f} s), single thread", w, text


def run(args, ranks, ClockSampler, peaks, cuda_sync):
    from vtl_b200 import capi
    dev = capi.Device(ranks.local_rank)
    ranks.attach(dev)
    sizes = tensor_sizes()
    rng = np.random.default_rng(4)
    big = rng.standard_normal(WIDTH * WIDTH, dtype=np.float32)
    small = rng.standard_normal(WIDTH, dtype=np.float32)
    params = [dev.to_device(big if n == WIDTH * WIDTH else small) for n in sizes]
    lens = [dev.ckpt_text_len(n) for n in sizes]
    texts = [dev.zeros((L,), np.uint8) for L in lens]
    n_total, text_total = sum(sizes), sum(lens)
    bytes_step = 4 * n_total + text_total

    def step():
        for p, n, t in zip(params, sizes, texts):
            dev.ckpt_encode_f32(p, n, t)

    cuda_sync(dev)
    sampler = ClockSampler(ranks.local_rank)
    if ranks.rank == 0:
        sampler.start()
    ranks.barrier()
    for _ in range(args.warmup):
        step()
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
    # the dominant kernel alone: the encode of one weight matrix, and the decode beside it
    evs = [(dev.event(), dev.event()) for _ in range(args.steps)]
    for i in range(args.steps):
        j = 2 * (i % LAYERS)
        dev.record(evs[i][0])
        dev.ckpt_encode_f32(params[j], sizes[j], texts[j])
        dev.record(evs[i][1])
    dev.sync()
    enc_ms = statistics.mean(dev.elapsed_ms(a, c) for a, c in evs)
    back = dev.zeros((WIDTH * WIDTH,), np.float32)
    t0 = time.perf_counter()
    for i in range(min(args.steps, 8)):
        dev.ckpt_decode_f32(texts[0], lens[0], back, sizes[0])  # blocks (it reports bad text)
    dec_ms = (time.perf_counter() - t0) * 1e3 / min(args.steps, 8)
    assert np.array_equal(back.numpy(), big), "decode(encode(w)) != w"
    assert dev.check_status() == 0

    # end to end: the text of every tensor lands in (pinned) host memory, as save_checkpoint needs it
    h_text = C.c_void_p()
    assert dev.lib.vtlb_host_alloc(max(lens), C.byref(h_text)) == 0

    def e2e_step():
        for p, n, t, L in zip(params, sizes, texts, lens):
            dev.ckpt_encode_f32(p, n, t)
            dev.d2h_raw(h_text.value, t, L)  # blocks until the text is on the host

    e2e_step()
    cuda_sync(dev)
    ranks.barrier()
    t0 = time.perf_counter()
    e2e_steps = max(1, min(args.steps, 5))
    for _ in range(e2e_steps):
        e2e_step()
    cuda_sync(dev)
    e2e_ms = ranks.max_f32((time.perf_counter() - t0) * 1e3) / e2e_steps
    clocks = sampler.stop() if ranks.rank == 0 else None
    dev.lib.vtlb_host_free(h_text)

    out = None
    if ranks.rank == 0:
        pk = peaks()
        ms_step = ms_total / args.steps
        enc_bytes = 4 * sizes[0] + lens[0]
        achieved = enc_bytes / (enc_ms * 1e-3) / 1e9
        out = {
            "metric": "checkpoint_encode_gb_per_s", "value": bytes_step * ranks.world / (ms_step * 1e-3) / 1e9,
            "unit": "GB/s", "n_gpus": ranks.world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32 -> f64 big-endian bytes -> base64 text (u8)", "data": "synthetic",
            "config": {"workload": "checkpoint payload encoding of baseline config 4's parameters: "
                                   "8 x (4096x4096 weight + 4096 bias) f32 ~N(0,1), the text format of the "
                                   "reference's save_checkpoint", "values": n_total, "text_bytes": text_total,
                       "parallelism": f"{ranks.world} replica(s), no collective",
                       "l2": "537 MB read and 1432 MB written per step, far beyond the 126 MB L2",
                       "values_per_s": n_total * ranks.world / (ms_step * 1e-3),
                       "decode_ms_per_weight_matrix_incl_validation_sync": dec_ms},
            "e2e": {"value": bytes_step * ranks.world / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "h2d_bytes_per_step": 0, "d2h_bytes_per_step": int(text_total), "ms_per_step": e2e_ms,
                    "note": "parameters live on the device; the text of each tensor is copied to pinned host memory"},
            "gpu_launches": int(launches), "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "ckpt_encode_kernel on one 4096x4096 weight matrix",
                         "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": achieved / pk["hbm_gbs"],
                         "traffic": None, "algorithmic_bytes_per_launch": enc_bytes,
                         "peak_source": f"hbm_gbs of {pk['_source']}", "kernel_ms": enc_ms},
        }
        if ranks.world == 1:
            gbs, cores, sample, w, text = cpu_sample()
            got = texts[0].numpy()[: lens[0]].tobytes().decode("ascii")
            assert got == text, "device text differs from the oracle's"
            out["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
    return out


def run_reference(args, ranks):
    """CPU arm: the oracle's encoder, each step one weight matrix."""
    if ranks.rank != 0:
        return None
    from oracle import checkpoint as ock
    rng = np.random.default_rng(4)
    w = rng.standard_normal(WIDTH * WIDTH, dtype=np.float32)
    for _ in range(args.warmup):
        ock.encode_payload(w)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        text = ock.encode_payload(w)
    ms_step = (time.perf_counter() - t0) * 1e3 / args.steps
    gbs = (4 * w.size + len(text)) / (ms_step * 1e-3) / 1e9
    sample = f"each step = one {WIDTH}x{WIDTH} weight matrix of the 16 tensors, single thread"
    out = {"impl": "reference", "metric": "checkpoint_encode_gb_per_s", "value": gbs, "unit": "GB/s",
           "n_gpus": ranks.world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "f32 -> f64 big-endian bytes -> base64 text (u8)", "data": "synthetic",
           "config": {"workload": "checkpoint payload encoding of baseline config 4's parameters, CPU oracle",
                      "values": int(w.size)},
           "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "port", "sample": sample},
           "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "gpu_launches": 0}
    return out
