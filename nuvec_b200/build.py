"""Builds libnuvec_cuda.so (the C-ABI CUDA backend) in-tree with nvcc for sm_100a.

Usage: python -m nuvec_b200.build [--force] [--verbose] [--timeline]

--timeline builds libnuvec_cuda_timeline.so instead: the same library with the few-row kernel's
%globaltimer records compiled in (-DNUVEC_TIMELINE), for `bench.py --timeline`.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libnuvec_cuda.so"
TIMELINE_LIB = PKG / "libnuvec_cuda_timeline.so"
SOURCES = ["runtime.cu", "quantize.cu", "qmv.cu", "qmm.cu", "qqmm.cu", "ops.cu", "moe.cu", "convert.cu", "attention.cu", "peer.cu", "comm_nccl.cpp"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
         "-Xcompiler", "-Wall", "-diag-suppress", "177"]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def stale(lib: Path = LIB) -> bool:
    if not lib.exists():
        return True
    t = lib.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.cpp")) + \
        [PKG.parent / "include" / "nuvec_cuda.h", Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False, timeline: bool = False) -> Path:
    lib = TIMELINE_LIB if timeline else LIB
    if not force and not stale(lib):
        return lib
    objs = []
    procs = []
    build_dir = PKG / "build" / "timeline" if timeline else PKG / "build"
    build_dir.mkdir(parents=True, exist_ok=True)
    extra = (["-Xptxas", "-v"] if verbose else []) + (["-DNUVEC_TIMELINE"] if timeline else [])
    for src in SOURCES:
        obj = build_dir / (src.rsplit(".", 1)[0] + ".o")
        cmd = [nvcc(), *ARCH, *FLAGS, *extra, "-x", "cu", "-c", str(CSRC / src), "-o", str(obj)]
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(str(obj))
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            failed = True
            sys.stderr.write(f"--- {src} ---\n{out}\n")
        elif verbose or out.strip():
            sys.stderr.write(f"--- {src} ---\n{out}\n")
    if failed:
        raise RuntimeError("nvcc failed")
    link = [nvcc(), *ARCH, "-shared", "-o", str(lib), *objs, "-lcudart", "-ldl"]
    subprocess.run(link, check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv, timeline="--timeline" in sys.argv))
