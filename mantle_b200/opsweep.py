"""Stand-alone operator sweep on one GPU: OP.DOT (square), OP.CONV2D and MAXPOOL2D, forward and
backward, timed with CUDA events through the C ABI.

    python -m mantle_b200.opsweep [--math tf32|tf32x3|fp32] [--iters 10]

Every timed call is preceded by a 256 MB device fill (larger than the 126 MB L2), so operands come
from HBM.  Prints one Markdown table row per operator: milliseconds, algorithmic TFLOP/s or GB/s.
"""
from __future__ import annotations

import argparse

import numpy as np

import mantle_b200 as mb
from mantle_b200 import OP


def timed(ctx, flush, fn, iters):
    fn()
    ctx.sync()
    total = 0.0
    for _ in range(iters):
        flush.zero()
        ctx.timer_start(0)
        fn()
        ctx.timer_stop(0)
        total += ctx.timer_ms(0)
    return total / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--math", choices=("tf32", "tf32x3", "fp32"), default="tf32")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--dot", type=int, nargs="*", default=[1024, 2048, 4096, 8192])
    args = ap.parse_args()
    mode = {"tf32": mb.MATH_TF32, "tf32x3": mb.MATH_TF32X3, "fp32": mb.MATH_FP32}[args.math]
    ctx = mb.Context(0, mode)
    rng = np.random.default_rng(0)
    flush = ctx.empty((64 * 1024 * 1024,))
    rows = []

    for s in args.dot:
        a = ctx.array(rng.normal(0, 1, (s, s)).astype(np.float32))
        b = ctx.array(rng.normal(0, 1, (s, s)).astype(np.float32))
        c, ug = ctx.empty((s, s)), ctx.array(rng.normal(0, 1, (s, s)).astype(np.float32))
        da, db = ctx.empty((s, s)), ctx.empty((s, s))
        fl = 2.0 * s ** 3
        for name, fn in (("DOT %d fwd" % s, lambda: ctx.forward_op(OP.DOT, c, a, b)),
                         ("DOT %d bwd A" % s, lambda: ctx.backward_op(0, OP.DOT, ug, a, b, grad=da, accumulate=False)),
                         ("DOT %d bwd B" % s, lambda: ctx.backward_op(1, OP.DOT, ug, a, b, grad=db, accumulate=False))):
            ms = timed(ctx, flush, fn, args.iters)
            rows.append((name, ms, "%.1f TFLOP/s" % (fl / ms / 1e9)))
        for t in (a, b, c, ug, da, db):
            t.free()

    N, C, K, H, W, R = 256, 64, 64, 56, 56, 3
    kw = dict(padding=(1, 1), stride=(1, 1), dilation=(1, 1))
    x = ctx.array(rng.normal(0, 1, (N, C, H, W)).astype(np.float32))
    w = ctx.array((rng.normal(0, 1, (K, C, R, R)) / 24.0).astype(np.float32))
    bias = ctx.array(np.zeros(K, np.float32))
    y, ug = ctx.empty((N, K, H, W)), ctx.array(rng.normal(0, 1, (N, K, H, W)).astype(np.float32))
    dx, dw, dbias = ctx.empty((N, C, H, W)), ctx.empty((K, C, R, R)), ctx.empty((K,))
    fl = 2.0 * N * K * C * H * W * R * R
    for name, fn in (("CONV2D 256x64x56x56 k3 fwd", lambda: ctx.forward_op(OP.CONV2D, y, x, w, bias, **kw)),
                     ("CONV2D bwd input", lambda: ctx.backward_op(0, OP.CONV2D, ug, x, w, bias, grad=dx, accumulate=False, **kw)),
                     ("CONV2D bwd kernel", lambda: ctx.backward_op(1, OP.CONV2D, ug, x, w, bias, grad=dw, accumulate=False, **kw))):
        ms = timed(ctx, flush, fn, args.iters)
        rows.append((name, ms, "%.1f TFLOP/s" % (fl / ms / 1e9)))
    ms = timed(ctx, flush, lambda: ctx.backward_op(2, OP.CONV2D, ug, x, w, bias, grad=dbias, accumulate=False, **kw), args.iters)
    rows.append(("CONV2D bwd bias", ms, "%.0f GB/s" % (N * K * H * W * 4 / ms / 1e6)))
    for t in (x, w, y, ug, dx, dw):
        t.free()

    N, C, H, W = 256, 64, 112, 112
    pk = dict(kernel_size=(2, 2), stride=(2, 2), padding=(0, 0), dilation=(1, 1))
    x = ctx.array(rng.normal(0, 1, (N, C, H, W)).astype(np.float32))
    y, idx = ctx.empty((N, C, H // 2, W // 2)), ctx.empty((N, C, H // 2, W // 2), np.int32)
    ug, dx = ctx.array(rng.normal(0, 1, (N, C, H // 2, W // 2)).astype(np.float32)), ctx.empty((N, C, H, W))
    n_in, n_out = N * C * H * W, N * C * H * W // 4
    ms = timed(ctx, flush, lambda: ctx.forward_op(OP.MAXPOOL2D, y, x, indices=idx, **pk), args.iters)
    rows.append(("MAXPOOL2D 256x64x112x112 fwd (+indices)", ms, "%.0f GB/s" % ((n_in + 2 * n_out) * 4 / ms / 1e6)))
    ms = timed(ctx, flush, lambda: ctx.backward_op(0, OP.MAXPOOL2D, ug, x, grad=dx, accumulate=False, indices=idx, **pk), args.iters)
    rows.append(("MAXPOOL2D bwd (from indices)", ms, "%.0f GB/s" % ((n_in + 2 * n_out) * 4 / ms / 1e6)))
    ms = timed(ctx, flush, lambda: ctx.backward_op(0, OP.MAXPOOL2D, ug, x, grad=dx, accumulate=False, **pk), args.iters)
    rows.append(("MAXPOOL2D bwd (reference form, re-scans X)", ms, "%.0f GB/s" % ((2 * n_in + n_out) * 4 / ms / 1e6)))

    print("| operator (%s) | ms | algorithmic rate |" % args.math)
    print("|---|---|---|")
    for name, ms, rate in rows:
        print("| %s | %.3f | %s |" % (name, ms, rate))
    print("device status", ctx.device_status())
    ctx.close()


if __name__ == "__main__":
    main()
