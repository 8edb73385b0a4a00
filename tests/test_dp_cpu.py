"""Data-parallel arithmetic on CPU ranks (gloo, world size 2): sharding the batch, summing the flat
gradients across ranks and applying Adam with grad_scale = 1/world reproduces the single-process
step on the whole batch.  The ranks compute with the CPU oracle; the reduction and the scaling are
what the GPU trainer does with NCCL (mantle_b200/host/trainer.cpp)."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch
    import torch.distributed as dist
    import oracle
    from test_oracle_kat import build_cnn
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    B = 8
    rng = np.random.default_rng(7)
    x = rng.uniform(0, 1, (B, 1, 28, 28)).astype(np.float32)
    y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, B)]
    shapes = [(16, 1, 5, 5), (16,), (32, 16, 5, 5), (32,), (1568, 10), (10,)]
    ws = [rng.uniform(-0.1, 0.1, s).astype(np.float32) for s in shapes]

    def make(batch):
        g = oracle.Graph()
        build_cnn(oracle, g, batch)
        m = oracle.Model(g)
        tr = [s for s in g.params() if s.trainable]
        for s, w in zip(tr, ws):
            m.set_tensor(s, w)
        return g, m, tr, oracle.Adam(m, lr=1e-3)

    lb = B // world
    g, m, tr, opt = make(lb)
    opt.grad_scale = 1.0 / world          # local losses are means over the local slice
    losses = []
    for step in range(3):
        loss = m.forward(x[rank * lb:(rank + 1) * lb], y[rank * lb:(rank + 1) * lb])
        opt.zero_grad(); m.backward()
        for s in tr:                       # the flat gradient arena, summed across ranks
            t = torch.from_numpy(m.grads[s.id])
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        opt.step()
        lt = torch.tensor([loss], dtype=torch.float64)
        dist.all_reduce(lt, op=dist.ReduceOp.SUM)
        losses.append(float(lt.item()) / world)   # mean of the per-rank mean losses
    if rank == 0:
        g1, m1, tr1, opt1 = make(B)
        ref = []
        for step in range(3):
            ref.append(m1.forward(x, y)); opt1.zero_grad(); m1.backward(); opt1.step()
        ok = np.allclose(losses, ref, rtol=1e-5, atol=1e-6)
        for s, s1 in zip(tr, tr1):
            ok = ok and np.allclose(m.tensors[s.id], m1.tensors[s1.id], rtol=1e-4, atol=1e-6)
        q.put((ok, losses, ref))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_data_parallel_step_equals_full_batch():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    ok, losses, ref = q.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert ok, (losses, ref)


def test_trainer_bucket_plan_matches_reverse_parameter_order():
    """The trainer exchanges a parameter's gradient once the lowest-numbered node reading it has run
    its backward; for the CNN that is classifier first, conv1 last (reverse of the flat span)."""
    sys.path.insert(0, str(ROOT))
    import oracle
    from test_oracle_kat import build_cnn
    g = oracle.Graph()
    build_cnn(oracle, g, 4)
    tr = [s for s in g.params() if s.trainable]
    first_reader = {}
    for i, n in enumerate(g.nodes):
        for s in n.inputs:
            first_reader.setdefault(s.id, i)
    order = sorted(range(len(tr)), key=lambda p: -first_reader[tr[p].id])  # backward visits nodes in reverse
    # Linear's bias (ADD, node 8) precedes its weight (DOT, node 7); a CONV2D node finishes W and b together
    assert order == [5, 4, 2, 3, 0, 1]
