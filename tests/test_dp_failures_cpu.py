"""Host-side failure handling of the data-parallel group, on CPU ranks.

The rendezvous of mtl_dp_init (libmantle_cuda.so, csrc/dp.cu) runs with a deadline.  Here every
rank is a child process that binds a stand-in collective library (tests/fake_nccl.c, built into a
temporary directory, rendezvous through files) and calls mtl_dp_probe -- the context-free form of
the same join.  Cases: everybody on time; one rank late but inside the deadline; one rank that never
starts.  In the last case every other rank must come back with MTL_ERR_COMM within the deadline
instead of hanging.  No GPU is involved and nothing here makes a GPU fault or hang."""
import ctypes as C
import multiprocessing as mp
import os
import subprocess
import time
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
MTL_OK, MTL_ERR_COMM = 0, 6


@pytest.fixture(scope="module")
def fake_nccl(tmp_path_factory, built):
    d = tmp_path_factory.mktemp("fake_nccl")
    so = d / "libfake_nccl.so"
    subprocess.run(["gcc", "-O1", "-shared", "-fPIC", "-fvisibility=hidden", "-o", str(so), str(ROOT / "tests" / "fake_nccl.c")],
                   check=True)
    return so


def _rank(rank, world, so, rdv, delay_s, timeout_ms, q):
    os.environ["MANTLE_NCCL_LIB"] = str(so)
    os.environ["FAKE_NCCL_DIR"] = str(rdv)
    lib = C.CDLL(str(ROOT / "mantle_b200" / "lib" / "libmantle_cuda.so"))
    lib.mtl_dp_get_unique_id.argtypes = [C.POINTER(C.c_uint8)]
    lib.mtl_dp_probe.argtypes = [C.POINTER(C.c_uint8), C.c_int32, C.c_int32, C.c_int32]
    uid = (C.c_uint8 * 128)()
    assert lib.mtl_dp_get_unique_id(uid) == MTL_OK
    time.sleep(delay_s)
    t0 = time.perf_counter()
    rc = lib.mtl_dp_probe(uid, rank, world, timeout_ms)
    q.put((rank, rc, time.perf_counter() - t0))


def _run(so, rdv, world, delays, timeout_ms, absent=()):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, world, so, rdv, delays.get(r, 0.0), timeout_ms, q))
             for r in range(world) if r not in absent]
    for p in procs:
        p.start()
    out = {}
    for _ in procs:
        rank, rc, dt = q.get(timeout=60)
        out[rank] = (rc, dt)
    for p in procs:
        p.join(timeout=30)
        assert p.exitcode == 0      # a rank whose helper thread is still blocked must still exit cleanly
    return out


def test_all_ranks_on_time(fake_nccl, tmp_path):
    out = _run(fake_nccl, tmp_path, 3, {}, 5000)
    assert {r: rc for r, (rc, _) in out.items()} == {0: MTL_OK, 1: MTL_OK, 2: MTL_OK}


def test_a_late_rank_inside_the_deadline_is_waited_for(fake_nccl, tmp_path):
    out = _run(fake_nccl, tmp_path, 3, {2: 1.0}, 8000)
    assert all(rc == MTL_OK for rc, _ in out.values())
    assert out[0][1] >= 0.5, "rank 0 must have waited for the late rank"


def test_a_missing_rank_ends_the_others_with_an_error_within_the_deadline(fake_nccl, tmp_path):
    out = _run(fake_nccl, tmp_path, 3, {}, 1500, absent=(1,))
    assert set(out) == {0, 2}
    for rank, (rc, dt) in out.items():
        assert rc == MTL_ERR_COMM, "rank %d returned %d" % (rank, rc)
        assert 1.0 <= dt < 6.0, "rank %d came back after %.2f s for a 1.5 s deadline" % (rank, dt)


def test_a_rank_later_than_the_deadline_fails_everywhere(fake_nccl, tmp_path):
    out = _run(fake_nccl, tmp_path, 2, {1: 2.5}, 1000)
    assert out[0][0] == MTL_ERR_COMM
    # the late rank finds rank 0's marker (the stand-in's files stay), so its own join may succeed; what
    # matters is that nobody blocks
    assert out[1][1] < 6.0
