"""Memory-safety run of the host-side code: the C oracle (oracle/mantle_oracle.c) and the C++ host
mirror (mantle_b200/host) are rebuilt with AddressSanitizer and UndefinedBehaviorSanitizer and the
CPU tests that exercise them -- the oracle's known answers and 100-step trajectories, the graph
builder and its shape rules, the layout operators' restatement, the checkpoint reader -- run again
in a child interpreter with the sanitizer runtimes preloaded.  Any out-of-bounds access, use after
free, signed overflow or misaligned access in that code ends the child with a report.  (Device code
cannot be run under these tools; the GPU tests guard it with exact comparisons and status words.)"""
import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _runtime(name):
    out = subprocess.run(["gcc", "-print-file-name=" + name], capture_output=True, text=True).stdout.strip()
    return out if out and os.path.isabs(out) and os.path.exists(out) else None


@pytest.mark.skipif(shutil.which("gcc") is None or _runtime("libasan.so") is None, reason="gcc with libasan is needed")
def test_oracle_and_host_mirror_under_asan_and_ubsan(tmp_path, built):
    san = ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-g", "-O1"]
    gomp = [p for p in Path("/usr/lib/gcc/x86_64-linux-gnu").glob("*/libgomp.spec")]
    omp = ["-fopenmp"] + (["-B" + str(gomp[0].parent) + "/"] if gomp else [])
    oracle_so = tmp_path / "libmantle_oracle_san.so"
    subprocess.run(["gcc"] + san + omp + ["-ffp-contract=off", "-march=x86-64-v3", "-fPIC", "-shared", "-o", str(oracle_so),
                                         str(ROOT / "oracle" / "mantle_oracle.c"), "-lm"], check=True)
    host_so = tmp_path / "libmantle_host_san.so"
    libdir = ROOT / "mantle_b200" / "lib"
    subprocess.run(["g++"] + san + ["-std=c++17", "-fPIC", "-shared", "-I", str(ROOT / "include"), "-o", str(host_so)] +
                   [str(p) for p in sorted((ROOT / "mantle_b200" / "host").glob("*.cpp"))] +
                   ["-L", str(libdir), "-lmantle_cuda", "-Wl,-rpath," + str(libdir)], check=True)
    env = dict(os.environ)
    env.update({
        "LD_PRELOAD": ":".join(p for p in (_runtime("libasan.so"), _runtime("libubsan.so")) if p),
        # the interpreter's own arenas are not of interest; stop at the first finding in our code
        "ASAN_OPTIONS": "detect_leaks=0:abort_on_error=1:halt_on_error=1",
        "UBSAN_OPTIONS": "halt_on_error=1:print_stacktrace=1",
        "MANTLE_ORACLE_LIB": str(oracle_so),
        "MANTLE_HOST_LIB": str(host_so),
        "OMP_NUM_THREADS": "4",
    })
    cmd = [sys.executable, "-m", "pytest", "-x", "-q", "-m", "not gpu", "-p", "no:cacheprovider",
           str(ROOT / "tests" / "test_oracle_kat.py"), str(ROOT / "tests" / "test_abi.py"),
           str(ROOT / "tests" / "test_layout_ops.py"), str(ROOT / "tests" / "test_checkpoint.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=1500, cwd=str(ROOT))
    tail = (r.stdout + r.stderr)[-4000:]
    assert r.returncode == 0, "sanitizer run failed:\n" + tail
    assert "passed" in r.stdout and "AddressSanitizer" not in tail and "runtime error" not in tail, tail
