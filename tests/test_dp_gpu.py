"""Data-parallel training on real GPUs (one process per GPU, NCCL through mtl_dp_*): the loss
trajectory of G ranks on slices of the global batch equals the single-GPU trajectory on the whole
batch within 1e-3 relative, and all ranks end with identical parameters.  Needs at least two
visible GPUs; skipped otherwise."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
pytestmark = pytest.mark.gpu

STEPS, GLOBAL_B = 12, 64


def _data():
    rng = np.random.default_rng(17)
    x = rng.uniform(0, 1, (STEPS, GLOBAL_B, 1, 28, 28)).astype(np.float32)
    y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, (STEPS, GLOBAL_B))]
    shapes = [(64, 1, 5, 5), (64,), (128, 64, 5, 5), (128,), (6272, 10), (10,)]
    ws = [(rng.uniform(-1, 1, s) / np.sqrt(max(int(np.prod(s[1:])), 16))).astype(np.float32) for s in shapes]
    return x, y, ws


def _tail_values(rank):
    return np.random.default_rng(100 + rank).normal(0, 1, 3001).astype(np.float32)


def _train(rank, world, uid, q):
    try:
        _train_body(rank, world, uid, q)
    except BaseException as e:  # the parent fails with the child's message instead of waiting for its time-out
        import traceback
        q.put((rank, "error", traceback.format_exc(), -1))
        raise


def _train_body(rank, world, uid, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import ctypes as C
    import mantle_b200 as mb
    from mantle_b200 import host_api, OP
    from test_oracle_kat import build_cnn

    import types
    Ns = types.SimpleNamespace(OP=OP, nn=host_api.nn, Graph=host_api.Graph)

    x, y, ws = _data()
    ctx = mb.Context(rank, mb.MATH_TF32X3)
    if world > 1:
        raw = (C.c_uint8 * mb._lib.MTL_DP_ID_BYTES)(*uid)
        ctx._check(ctx.lib.mtl_dp_init(ctx.handle, raw, rank, world))
    lb = GLOBAL_B // world
    g = host_api.Graph()
    build_cnn(Ns, g, lb, 64, 128)
    m = host_api.Model(ctx, g)
    tr = [s for s in g.params() if s.trainable]
    for s, w in zip(tr, ws):
        m.set_tensor(s, w)
    trainer = host_api.Trainer(m, host_api.Adam(m, lr=1e-3), use_graph=True)
    losses = [trainer.step(x[i, rank * lb:(rank + 1) * lb], y[i, rank * lb:(rank + 1) * lb]) for i in range(STEPS)]
    params = [m.tensor(s) for s in tr]
    # the direct exchange of a step's last bucket, called by hand: two exchanges in a row of rank-specific values
    tail_on = int(ctx.lib.mtl_dp_tail_exchange_enabled(ctx.handle))
    tail = None
    if world > 1:
        v = ctx.array(_tail_values(rank))
        for _ in range(2):
            ctx._check(ctx.lib.mtl_dp_allreduce_tail(ctx.handle, v.ptr, v.size))
        ctx.sync()
        tail = v.numpy()
    status = ctx.device_status()
    trainer.close()
    q.put((rank, losses, params, status, tail_on, tail))
    ctx.close()


def _run(world):
    import torch.multiprocessing as mp
    import ctypes as C
    import mantle_b200 as mb
    uid = None
    if world > 1:
        raw = (C.c_uint8 * mb._lib.MTL_DP_ID_BYTES)()
        assert mb.cuda_lib().mtl_dp_get_unique_id(raw) == 0, "NCCL is not loadable"
        uid = list(raw)
    mpc = mp.get_context("spawn")
    q = mpc.Queue()
    procs = [mpc.Process(target=_train, args=(r, world, uid, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = []
    try:
        for _ in range(world):
            item = q.get(timeout=180)
            assert item[1] != "error", "rank %d failed:\n%s" % (item[0], item[2])
            out.append(item)
    finally:
        for p in procs:
            p.join(timeout=60)
            if p.is_alive():
                p.kill()
    assert all(p.exitcode == 0 for p in procs)
    return sorted(out, key=lambda t: t[0])


@pytest.mark.parametrize("world", (2, 4, 8))
def test_data_parallel_trajectory_equals_single_gpu(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip("needs %d GPUs" % world)
    os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
    single = _run(1)[0]
    ranks = _run(world)
    assert all(r[3] == 0 for r in ranks) and single[3] == 0
    # the global loss is the mean of the per-rank mean losses (equal slice sizes)
    got = np.mean([r[1] for r in ranks], axis=0)
    want = np.asarray(single[1])
    assert np.allclose(got, want, rtol=1e-3, atol=1e-6), (got, want)
    assert got[-1] < got[0]
    for r in ranks[1:]:                       # replicas stay identical
        for a, b in zip(ranks[0][2], r[2]):
            assert np.array_equal(a, b)
    for a, b in zip(ranks[0][2], single[2]):  # and close to the single-GPU parameters
        assert np.linalg.norm(a - b) <= 2e-2 * np.linalg.norm(b) + 1e-6
    # ranks of one machine exchange the last bucket directly; the sum runs in rank order on every rank
    assert all(r[4] == 1 for r in ranks), [r[4] for r in ranks]
    want = np.zeros(3001, np.float32)
    for r in range(world):
        want = want + _tail_values(r)
    first = want.copy()
    want = np.zeros(3001, np.float32)
    for r in range(world):
        want = want + first
    for r in ranks:
        assert np.array_equal(r[5], want)


def test_direct_exchange_of_every_bucket_opt_in(monkeypatch):
    """MANTLE_DP_BUCKET_EXCHANGE=1: the buckets that overlap the backward pass travel through the library's own
    exchange kernel as well (on the communication stream) instead of NCCL; same trajectory, identical replicas."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    single = _run(1)[0]
    monkeypatch.setenv("MANTLE_DP_BUCKET_EXCHANGE", "1")
    ranks = _run(2)
    assert all(r[3] == 0 and r[4] == 1 for r in ranks)
    got = np.mean([r[1] for r in ranks], axis=0)
    assert np.allclose(got, np.asarray(single[1]), rtol=1e-3, atol=1e-6)
    for a, b in zip(ranks[0][2], ranks[1][2]):
        assert np.array_equal(a, b)


def _visible_gpus():
    import ctypes as C
    try:
        rt = C.CDLL("libcudart.so")
    except OSError:
        try:
            rt = C.CDLL("libcudart.so.12")
        except OSError:
            return 0
    n = C.c_int(0)
    return n.value if rt.cudaGetDeviceCount(C.byref(n)) == 0 else 0


def test_two_contexts_on_two_devices_from_one_thread():
    """Every entry point makes its context's device current for the call and restores the caller's: one
    host thread can drive contexts on different GPUs in turn (allocation, operators, a captured step)
    and each result lands on, and is computed by, its own device."""
    if _visible_gpus() < 2:
        pytest.skip("needs two visible GPUs")
    import mantle_b200 as mb
    from mantle_b200 import OP
    import oracle
    c0, c1 = mb.Context(0), mb.Context(1)
    rng = np.random.default_rng(5)
    a = rng.normal(0, 1, (256, 128)).astype(np.float32)
    b = rng.normal(0, 1, (128, 256)).astype(np.float32)
    outs = []
    for step in range(3):                       # interleaved calls on the two contexts
        for ctx, scale in ((c0, 1.0), (c1, 2.0)):
            da, db = ctx.array(a * np.float32(scale)), ctx.array(b)
            out = ctx.empty((256, 256))
            ctx.forward_op(OP.DOT, out, da, db)
            outs.append((scale, out))
    want = oracle.dot(a, b)
    for scale, out in outs:
        got = out.numpy()
        assert float(np.max(np.abs(got - scale * want)) / np.max(np.abs(want))) < 3e-5
    assert c0.device_status() == 0 and c1.device_status() == 0
    c1.close(); c0.close()
