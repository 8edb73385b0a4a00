"""Builds libmantle_cuda.so (sm_100a) and libmantle_host.so in-tree with nvcc / g++.

    python -m mantle_b200.build            # build what is out of date
    python -m mantle_b200.build --force    # rebuild everything

The CUDA library holds the kernels and the C ABI declared in include/mantle_cuda.h; the host
library holds the C++ mirror of Mantle's graph executor and Adam (mantle_b200/host), which calls
the C ABI only.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
HOST = PKG / "host"
LIBDIR = PKG / "lib"
OBJDIR = PKG / "build"

CUDA_LIB = LIBDIR / "libmantle_cuda.so"
HOST_LIB = LIBDIR / "libmantle_host.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found: libmantle_cuda.so cannot be built")
    return exe


def _newer(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(d.stat().st_mtime <= t for d in deps)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(cmd), proc.stdout, proc.stderr))


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    srcs = sorted(CSRC.glob("*.cu"))
    hdrs = sorted(CSRC.glob("*.cuh")) + [ROOT / "include" / "mantle_cuda.h"]
    OBJDIR.mkdir(exist_ok=True)
    LIBDIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    jobs = []
    objs = []
    for s in srcs:
        o = OBJDIR / (s.stem + ".o")
        objs.append(o)
        if force or not _newer(o, [s] + hdrs):
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", str(s), "-o", str(o)]
            jobs.append(cmd)
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            list(ex.map(_run, jobs))
    if force or jobs or not _newer(CUDA_LIB, objs):
        _run([nvcc, "-shared", "-o", str(CUDA_LIB)] + [str(o) for o in objs] + ["-ldl"])
    return CUDA_LIB


def build_host(force: bool = False) -> Path:
    srcs = sorted(HOST.glob("*.cpp"))
    hdrs = sorted(HOST.glob("*.hpp")) + [ROOT / "include" / "mantle_cuda.h"]
    if not srcs:
        return HOST_LIB
    LIBDIR.mkdir(exist_ok=True)
    if force or not _newer(HOST_LIB, srcs + hdrs + [CUDA_LIB]):
        cxx = shutil.which("g++") or "g++"
        _run([cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-I", str(ROOT / "include"),
              "-o", str(HOST_LIB)] + [str(s) for s in srcs] +
             ["-L", str(LIBDIR), "-lmantle_cuda", "-Wl,-rpath,$ORIGIN"])
    return HOST_LIB


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_host(force)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    build_all(a.force, a.verbose)
    print(CUDA_LIB)
    print(HOST_LIB if HOST_LIB.exists() else "(no host library sources yet)")
