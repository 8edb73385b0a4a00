"""The allocation-free whole-tensor reduction (mtl_reduce_all_static) against the regular entry
point (mtl_reduce_fwd), through the C ABI, on two consecutive calls.

The static variant serves callers that cannot allocate device memory when they reduce (all GPU
memory already owned by another pool, or no tolerance for the wait an allocation may cause); it
keeps its per-block partials in an array built into the library instead of the context workspace.
This file is named to be collected last, so that a run stopping at the first failure has already
executed every other test."""
import numpy as np
import pytest

import mantle_b200 as mb
from mantle_b200 import OP

pytestmark = pytest.mark.gpu


def _reduce(ctx, fn_static, op, x_dev, n):
    out = ctx.empty((1,))
    if fn_static:
        ctx._check(ctx.lib.mtl_reduce_all_static(ctx.handle, op, out.ptr, x_dev.ptr, n))
    else:
        ctx.forward_op(op, out, x_dev)
    return out.numpy()


def test_static_reduce_matches_regular_twice(ctx):
    rng = np.random.default_rng(21)
    for call, n in enumerate((1_000_003, 77)):          # two calls in a row share the static array
        x = rng.normal(0, 1, n).astype(np.float32)
        xd = ctx.array(x)
        for op in (OP.SUM, OP.MEAN, OP.MAX):
            want = _reduce(ctx, False, op, xd, n)
            got = _reduce(ctx, True, op, xd, n)
            # same kernels and launch shape on both paths: the tolerance of the other reduction tests
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-5, err_msg="call %d op %d" % (call, op))
            ref = {OP.SUM: x.sum(dtype=np.float64), OP.MEAN: x.mean(dtype=np.float64), OP.MAX: x.max()}[op]
            np.testing.assert_allclose(got[0], ref, rtol=1e-4, atol=1e-3)


def test_static_reduce_rejects_oversize_and_bad_ops(ctx):
    a = ctx.zeros((8,))
    out = ctx.empty((1,))
    L, h = ctx.lib, ctx.handle
    assert L.mtl_reduce_all_static(h, OP.SUM, out.ptr, a.ptr, (1 << 28) + 1) == 1
    assert b"at most" in L.mtl_last_error(h) or b"handles" in L.mtl_last_error(h)
    assert L.mtl_reduce_all_static(h, OP.SUM, out.ptr, a.ptr, 0) == 1
    assert L.mtl_reduce_all_static(h, OP.DOT, out.ptr, a.ptr, 8) == 1
    assert L.mtl_reduce_all_static(h, OP.SUM, None, a.ptr, 8) == 1
