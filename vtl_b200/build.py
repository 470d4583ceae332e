"""Builds libvtlb200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

    python -m vtl_b200.build [--force] [--verbose]

Each .cu file under csrc/ is compiled to an object (in parallel) and the objects
are linked into vtl_b200/libvtlb200.so.  Objects are rebuilt when their source
or any header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libvtlb200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall,-Wno-unused-function",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: libvtlb200.so cannot be built")


def _sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))


def _compile(src: str, obj: str, verbose: bool) -> str:
    extra = os.environ.get("VTLB_NVCC_EXTRA", "").split()  # e.g. -DVTLB_PAIR_STAGES=7 for tuning runs
    cmd = [_nvcc(), *NVCC_FLAGS, *extra, "-ccbin", "g++", "-I", os.path.join(HERE, "..", "include"),
           "-c", src, "-o", obj]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{p.stdout}\n{p.stderr}")
    log = p.stdout + p.stderr
    with open(obj + ".log", "w") as f:
        f.write(log)
    if verbose:
        print(log)
    return log


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    hdr_time = max((os.path.getmtime(h) for h in _headers()), default=0)
    jobs = []
    objs = []
    for src in _sources():
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or os.path.getmtime(obj) < max(
            os.path.getmtime(src), hdr_time)
        if stale:
            jobs.append((src, obj))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for fut in [ex.submit(_compile, s, o, verbose) for s, o in jobs]:
                fut.result()
    if jobs or not os.path.exists(LIB):
        cmd = [_nvcc(), "-shared", "-o", LIB, *objs, "-ccbin", "g++", "-ldl"]
        p = subprocess.run(cmd, capture_output=True, text=True)
        if p.returncode != 0:
            raise RuntimeError(f"link failed:\n{p.stdout}\n{p.stderr}")
    _build_host(force or bool(jobs), verbose)
    return LIB


HOST_LIB = os.path.join(HERE, "libvtl_host.so")


def _build_host(force: bool, verbose: bool) -> str:
    """The C++ host mirror (csrc/host): plain g++, linked against libvtlb200.so only."""
    hdir = os.path.join(CSRC, "host")
    srcs = sorted(glob.glob(os.path.join(hdir, "*.cpp")))
    deps = srcs + glob.glob(os.path.join(hdir, "*.h*")) + [os.path.join(HERE, "..", "include", "vtlb.h")]
    if not force and os.path.exists(HOST_LIB) and os.path.getmtime(HOST_LIB) >= max(map(os.path.getmtime, deps)):
        return HOST_LIB
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-fvisibility=default", "-o", HOST_LIB, *srcs,
           "-L", HERE, "-lvtlb200", "-Wl,-rpath,$ORIGIN"]
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError(f"host library build failed:\n{p.stdout}\n{p.stderr}")
    if verbose:
        print(p.stdout, p.stderr)
    return HOST_LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
