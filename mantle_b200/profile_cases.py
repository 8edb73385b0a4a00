"""Small, fixed workloads for profiling one kernel at a time with Nsight Compute:

    python -m mantle_b200.profile_cases <case> [--math tf32|tf32x3|fp32] [--reps 3]
    ncu --section SpeedOfLight --section MemoryWorkloadAnalysis --clock-control none \\
        -k regex:<kernel> -s 1 -c 1 python -m mantle_b200.profile_cases <case>

Each case runs one operator (forward and, where named so, backward) `reps` times on seeded data
through the C ABI and prints the device status.  Inputs are larger than the 126 MB L2 but hold at
most about 2 GB on the device, so that a capture ends within a minute or two.

cases: dot1024 dot2048 dot4096 dot8192 | conv_sweep (CONV2D [256,64,56,56] k3, fwd + dX + dW + db) |
       conv2 (CONV2D [2048,64,14,14] -> 128, k5, the CNN's second layer) | conv1 (first layer, fused
       CONV2D+RELU+MAXPOOL2D forward and its backward from the pooled gradient) |
       pool (MAXPOOL2D 2x2 on [128,64,112,112], forward and both backward forms) |
       linear (Linear 6272 -> 10 at batch 2048, one launch each way) | adam (64 Mi parameters) |
       add relu (64 Mi elements) | sum max (256 Mi elements)
"""
from __future__ import annotations

import argparse
import ctypes as C

import numpy as np

import mantle_b200 as mb
from mantle_b200 import OP


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--math", choices=("tf32", "tf32x3", "fp32"), default="tf32")
    ap.add_argument("--reps", type=int, default=3)
    a = ap.parse_args()
    ctx = mb.Context(0, {"tf32": mb.MATH_TF32, "tf32x3": mb.MATH_TF32X3, "fp32": mb.MATH_FP32}[a.math])
    rng = np.random.default_rng(0)
    L, h = ctx.lib, ctx.handle

    def rnd(shape, scale=1.0):
        return ctx.array((rng.standard_normal(shape, dtype=np.float32) * np.float32(scale)))

    case = a.case
    if case.startswith("dot"):
        s = int(case[3:])
        x, w, ug, out = rnd((s, s)), rnd((s, s)), rnd((s, s)), ctx.empty((s, s))
        for _ in range(a.reps):
            ctx.forward_op(OP.DOT, out, x, w)
            ctx.backward_op(0, OP.DOT, ug, x, w, grad=out, accumulate=False)
            ctx.backward_op(1, OP.DOT, ug, x, w, grad=out, accumulate=False)
    elif case in ("conv_sweep", "conv2"):
        n, c, hw, k, r, pad = (256, 64, 56, 64, 3, 1) if case == "conv_sweep" else (2048, 64, 14, 128, 5, 2)
        x, w, b = rnd((n, c, hw, hw)), rnd((k, c, r, r), 0.05), rnd((k,))
        ug = rnd((n, k, hw, hw))
        y, dx, dw, db = ctx.empty((n, k, hw, hw)), ctx.empty((n, c, hw, hw)), ctx.empty((k, c, r, r)), ctx.empty((k,))
        kw = dict(padding=(pad, pad))
        for _ in range(a.reps):
            ctx.forward_op(OP.CONV2D, y, x, w, b, **kw)
            ctx.backward_op(0, OP.CONV2D, ug, x, w, b, grad=dx, accumulate=False, **kw)
            ctx.backward_op(1, OP.CONV2D, ug, x, w, b, grad=dw, accumulate=False, **kw)
            ctx.backward_op(2, OP.CONV2D, ug, x, w, b, grad=db, accumulate=False, **kw)
    elif case == "conv1":
        n = 2048
        x = ctx.array(rng.uniform(0, 1, (n, 1, 28, 28)).astype(np.float32))
        w, b = rnd((64, 1, 5, 5), 0.2), rnd((64,), 0.1)
        pv, pi, tw = ctx.empty((n, 64, 14, 14)), ctx.empty((n, 64, 14, 14), np.int32), ctx.empty((n, 14, 14, 64))
        pg, dw, db = rnd((n, 64, 14, 14)), ctx.empty((64, 1, 5, 5)), ctx.empty((64,))
        d = mb.conv_desc(n, 1, 28, 28, 64, 5, 5, (2, 2), (1, 1), (1, 1))
        pd = mb.conv_desc(n, 64, 28, 28, 1, 2, 2, (0, 0), (2, 2), (1, 1))
        for _ in range(a.reps):
            ctx._check(L.mtl_conv2d_fwd_act_pool_cl(h, pv.ptr, pi.ptr, tw.ptr, x.ptr, None, w.ptr, b.ptr, C.byref(d), int(OP.RELU), C.byref(pd)))
            ctx._check(L.mtl_conv2d_bwd_pooled(h, None, dw.ptr, db.ptr, pg.ptr, pi.ptr, pv.ptr, x.ptr, None, w.ptr, C.byref(d), int(OP.RELU),
                                               C.byref(pd), 0, 0, 0))
    elif case == "pool":
        n, c, hw = 128, 64, 112
        x, ug = rnd((n, c, hw, hw)), rnd((n, c, hw // 2, hw // 2))
        y, idx, dx = ctx.empty((n, c, hw // 2, hw // 2)), ctx.empty((n, c, hw // 2, hw // 2), np.int32), ctx.empty((n, c, hw, hw))
        for _ in range(a.reps):
            ctx.forward_op(OP.MAXPOOL2D, y, x, kernel_size=(2, 2), indices=idx)
            ctx.backward_op(0, OP.MAXPOOL2D, ug, x, grad=dx, accumulate=False, kernel_size=(2, 2), indices=idx)
            ctx.backward_op(0, OP.MAXPOOL2D, ug, x, grad=dx, accumulate=False, kernel_size=(2, 2))
    elif case == "linear":
        m, k, n = 2048, 6272, 10
        x, w, b, ug = rnd((m, k)), rnd((k, n), 0.01), rnd((n,)), rnd((m, n))
        y, dx, dw, db = ctx.empty((m, n)), ctx.empty((m, k)), ctx.empty((k, n)), ctx.empty((n,))
        for _ in range(a.reps):
            ctx._check(L.mtl_linear_fwd(h, y.ptr, x.ptr, w.ptr, b.ptr, m, k, n))
            ctx._check(L.mtl_linear_bwd(h, dx.ptr, dw.ptr, db.ptr, ug.ptr, x.ptr, w.ptr, m, k, n, 0, 0, 0))
    elif case == "adam":
        n = 64 << 20
        p, g, m, v = rnd((n,)), rnd((n,), 0.01), ctx.zeros((n,)), ctx.zeros((n,))
        for t in range(a.reps):
            ctx.adam_step(p, g, m, v, n, 1e-3, 0.9, 0.999, 1e-8, t + 1)
    elif case in ("add", "relu"):
        n = 64 << 20
        x, y, out = rnd((n,)), rnd((n,)), ctx.empty((n,))
        for _ in range(a.reps):
            if case == "add":
                ctx.forward_op(OP.ADD, out, x, y)
            else:
                ctx.forward_op(OP.RELU, out, x)
                ctx.backward_op(0, OP.RELU, y, x, grad=out, accumulate=False)
    elif case in ("sum", "max"):
        n = 256 << 20
        x, out = rnd((n,)), ctx.empty((1,))
        for _ in range(a.reps):
            ctx.forward_op(OP.SUM if case == "sum" else OP.MAX, out, x)
    else:
        raise SystemExit("unknown case %r" % case)
    ctx.sync()
    print("case %s (%s): device status %d, %d kernel launches" % (case, a.math, ctx.device_status(), ctx.launch_count()))
    ctx.close()


if __name__ == "__main__":
    main()
