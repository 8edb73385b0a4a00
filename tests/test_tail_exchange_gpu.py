"""The direct exchange of a step's last gradient bucket (mtl_dp_allreduce_tail), exercised on ONE GPU by its
self-test entry point: the ranks of a group run as the block rows of one cooperative launch, each with its own
exchange buffer, and push / collect exactly as the ranks of a real group do.  Checked: the rank-ordered fp32
sum, bit for bit, on every rank, over several exchanges in a row (both buffer halves, step numbers advancing);
and a rank that never pushes, with a 2 ms budget: the others give up, the status word reads MTL_ERR_TIMEOUT,
their values are untouched and the context goes on working.  (Between processes on several GPUs the same
kernel body is covered by tests/test_dp_gpu.py.)"""
import numpy as np
import pytest

import mantle_b200 as mb

pytestmark = pytest.mark.gpu
MTL_ERR_TIMEOUT = 5


@pytest.fixture(scope="module")
def ctx():
    c = mb.Context(0)
    yield c
    c.close()


def rank_ordered_sums(vals, steps):
    cur = [v.copy() for v in vals]
    for _ in range(steps):
        s = np.zeros_like(cur[0])
        for v in cur:
            s = s + v
        cur = [s.copy() for _ in cur]
    return cur


@pytest.mark.parametrize("world,n,steps", [(2, 1, 1), (2, 1664, 3), (4, 3001, 2), (8, 1664, 4), (8, 16384, 2)])
def test_emulated_ranks_get_the_rank_ordered_sum(ctx, world, n, steps):
    rng = np.random.default_rng(world * 1000 + n)
    vals = [rng.normal(0, 1, n).astype(np.float32) for _ in range(world)]
    g = ctx.array(np.stack(vals))
    ctx._check(ctx.lib.mtl_selftest_tail_exchange(ctx.handle, g.ptr, world, n, steps, -1, 2_000_000))
    assert ctx.device_status() == 0
    got = g.numpy()
    want = rank_ordered_sums(vals, steps)
    for r in range(world):
        assert np.array_equal(got[r], want[r]), r


def test_a_silent_rank_ends_as_a_status_code(ctx):
    world, n = 4, 1000
    rng = np.random.default_rng(5)
    vals = [rng.normal(0, 1, n).astype(np.float32) for _ in range(world)]
    g = ctx.array(np.stack(vals))
    ctx._check(ctx.lib.mtl_selftest_tail_exchange(ctx.handle, g.ptr, world, n, 1, 2, 2000))
    assert ctx.device_status() == MTL_ERR_TIMEOUT
    assert np.array_equal(g.numpy(), np.stack(vals))      # nobody summed anything
    assert ctx.device_status() == 0                        # reading cleared it
    # the context still works
    ctx._check(ctx.lib.mtl_selftest_tail_exchange(ctx.handle, g.ptr, world, n, 1, -1, 2_000_000))
    assert ctx.device_status() == 0
    assert np.array_equal(g.numpy()[0], rank_ordered_sums(vals, 1)[0])
