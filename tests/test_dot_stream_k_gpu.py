"""The stream-K schedule of the tensor-core DOT kernel (an opt-in, MANTLE_GEMM_SPLITK=1), in a child
process because the switch is read when the library is first used: all three products, both
arithmetic modes, shapes whose tiles are split over two to four CTAs, against float64; and the
result must not depend on scheduling (two runs give identical bits)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHILD = r'''
import sys
import numpy as np
sys.path.insert(0, %r)
import mantle_b200 as mb
from mantle_b200 import OP
ctx = mb.Context(0)
rng = np.random.default_rng(3)
for (M, K, N) in ((1024, 1024, 1024), (512, 2048, 384), (2048, 512, 2048), (640, 4096, 896)):
    a = rng.normal(0, 1, (M, K)).astype(np.float32); b = rng.normal(0, 1, (K, N)).astype(np.float32)
    ug = rng.normal(0, 1, (M, N)).astype(np.float32)
    want = (a.astype(np.float64) @ b, ug.astype(np.float64) @ b.T.astype(np.float64), a.T.astype(np.float64) @ ug)
    da, db, dug = ctx.array(a), ctx.array(b), ctx.array(ug)
    for mode, tol in ((mb.MATH_TF32X3, 3e-5), (mb.MATH_TF32, 4e-3)):
        ctx.set_math_mode(mode)
        outs = []
        for rep in range(2):
            c, ga, gb = ctx.empty((M, N)), ctx.empty((M, K)), ctx.empty((K, N))
            ctx.forward_op(OP.DOT, c, da, db)
            ctx.backward_op(0, OP.DOT, dug, da, db, grad=ga, accumulate=False)
            ctx.backward_op(1, OP.DOT, dug, da, db, grad=gb, accumulate=False)
            outs.append((c.numpy(), ga.numpy(), gb.numpy()))
        for g, w, what in zip(outs[0], want, ("C", "dA", "dB")):
            e = float(np.max(np.abs(g - w)) / np.max(np.abs(w)))
            assert e < tol, (M, K, N, mode, what, e)
        for x, y in zip(outs[0], outs[1]):
            assert np.array_equal(x, y), "stream-K result depends on scheduling"
        init = rng.normal(0, 1, (K, N)).astype(np.float32)
        gacc = ctx.array(init)
        ctx.backward_op(1, OP.DOT, dug, da, db, grad=gacc, accumulate=True)
        assert float(np.max(np.abs(gacc.numpy() - (init + want[2]))) / np.max(np.abs(want[2]))) < tol
    assert ctx.device_status() == 0
print("CHILD_OK")
'''


def test_stream_k_schedule_matches_float64_and_is_deterministic():
    env = dict(os.environ, MANTLE_GEMM_SPLITK="1")
    r = subprocess.run([sys.executable, "-c", CHILD % str(ROOT)], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "CHILD_OK" in r.stdout, (r.stdout + r.stderr)[-3000:]
