"""Parity of every CUDA entry point with the CPU oracle on the same seeded inputs, called through
the C ABI (mantle_b200.Context.forward_op / backward_op are thin ctypes wrappers).

Tolerances: the reference's own `almost` comparison is rtol = atol = 1e-5
(tests/testing_utils.mojo:16-27); that is used for everything computed in fp32 on CUDA cores.
Tensor-core results are held to rtol 1e-4 / atol 1e-5 in 3xTF32 mode and rtol 5e-3 in plain TF32
mode; for long reductions the absolute part is scaled by the largest output magnitude, because the
tensor core's fp32 accumulation truncates and its error grows with the reduction length
(normalised max error < 3e-5 in 3xTF32 mode, < 4e-3 in TF32 mode, both checked).  Max-pool values, argmax
indices and shapes are compared exactly; MTL_MATH_FP32 DOT is compared bit-for-bit."""
import numpy as np
import pytest

import mantle_b200 as mb
import oracle
from mantle_b200 import OP
from helpers import assert_close, cases, golden

pytestmark = pytest.mark.gpu


def run_fwd(ctx, op, out_shape, *ts, **attrs):
    d = [ctx.array(t) for t in ts]
    res = ctx.empty(out_shape)
    ctx.forward_op(op, res, *d, **attrs)
    return res.numpy()


def run_bwd(ctx, tensor_id, op, ug, *ts, grad_shape, init=None, accumulate=True, **attrs):
    d = [ctx.array(t) for t in ts]
    grad = ctx.zeros(grad_shape) if init is None else ctx.array(init)
    dug = ctx.array(ug)
    ctx.backward_op(tensor_id, op, dug, *d, grad=grad, accumulate=accumulate, **attrs)
    return grad.numpy()


# ------------------------------------------------------------------ elementwise ----------------

BIN = {"add": OP.ADD, "sub": OP.SUB, "mul": OP.MUL, "div": OP.DIV}


def test_binary_forward_backward(ctx):
    z = golden("ops")
    rng = np.random.default_rng(1)
    for name in cases(z, "bin_"):
        f = lambda k: z["bin_%s__%s" % (name, k)]
        op = BIN[name[:3]]
        a, b, ug = f("a"), f("b"), f("ug")
        want = oracle.binary_fwd(op, a, b)
        assert_close(run_fwd(ctx, op, want.shape, a, b), want, what=name)
        assert_close(want, f("c"), what=name + " (torch)")
        for tid, t in ((0, a), (1, b)):
            init = rng.normal(0, 1, t.shape).astype(np.float32)
            want_g = oracle.binary_bwd(op, tid, ug, a, b, grad=init.copy())
            got = run_bwd(ctx, tid, op, ug, a, b, grad_shape=t.shape, init=init)
            assert_close(got, want_g, 1e-5, 1e-4, "%s d%d accumulate" % (name, tid))
            got = run_bwd(ctx, tid, op, ug, a, b, grad_shape=t.shape, init=init, accumulate=False)
            assert_close(got, oracle.binary_bwd(op, tid, ug, a, b), 1e-5, 1e-4, "%s d%d overwrite" % (name, tid))


def test_scalar_operand_paths(ctx):
    # a [1]-shaped operand selects the tensor-scalar path (tensorutils.mojo:266-269)
    rng = np.random.default_rng(2)
    t = rng.normal(0, 1, (33, 7)).astype(np.float32)  # odd size: exercises the non-vector tail
    s = np.array([1.7], np.float32)
    for op in BIN.values():
        assert_close(run_fwd(ctx, op, t.shape, t, s), oracle.binary_fwd(op, t, s))
        assert_close(run_fwd(ctx, op, t.shape, s, t), oracle.binary_fwd(op, s, t))
    ug = rng.normal(0, 1, t.shape).astype(np.float32)
    # gradient of a trainable [1] operand: everything sums into one element
    assert_close(run_bwd(ctx, 1, OP.ADD, ug, t, s, grad_shape=(1,)), oracle.binary_bwd(OP.ADD, 1, ug, t, s), 1e-5, 1e-4)
    assert_close(run_bwd(ctx, 1, OP.DIV, ug, t, s, grad_shape=(1,)), oracle.binary_bwd(OP.DIV, 1, ug, t, s), 1e-4, 1e-4)


UNARY = {"exp": (OP.EXP, {}), "log": (OP.LOG, {}), "sigmoid": (OP.SIGMOID, {}), "relu": (OP.RELU, {}),
         "tanh": (OP.TANH, {}), "pow2": (OP.POW, {"exponent": 2}), "pow3": (OP.POW, {"exponent": 3}),
         "leakyrelu": (OP.LEAKYRELU, {"negative_slope": 0.1}), "clip": (OP.CLIP, {"min": -0.3, "max": 0.4})}


def test_unary_forward_backward(ctx):
    z = golden("ops")
    for name, (op, kw) in UNARY.items():
        x, ug = z["un_%s__x" % name], z["un_%s__ug" % name]
        assert_close(run_fwd(ctx, op, x.shape, x, **kw), oracle.forward_op(op, x, **kw), what=name)
        init = np.full(x.shape, 0.5, np.float32)
        want = oracle.backward_op(0, op, ug, x, grad=init.copy(), **kw)
        assert_close(run_bwd(ctx, 0, op, ug, x, grad_shape=x.shape, init=init, **kw), want, what=name + " bwd")
        assert_close(run_bwd(ctx, 0, op, ug, x, grad_shape=x.shape, init=init, accumulate=False, **kw),
                     oracle.backward_op(0, op, ug, x, **kw), what=name + " bwd overwrite")


def test_fma_forward_and_three_backward_arms(ctx):
    """FMA (basics.mojo:759-817) at the shape of tests/python/test_ops_torch.mojo:881 (an odd element
    count, so the vector tail runs too) and on a tiny tensor."""
    rng = np.random.default_rng(12)
    for shape in ((87, 73, 84), (2, 3)):
        t1, t2, t3, ug = (rng.normal(0, 1, shape).astype(np.float32) for _ in range(4))
        got = run_fwd(ctx, OP.FMA, shape, t1, t2, t3)
        assert_close(got, oracle.forward_op(OP.FMA, t1, t2, t3), 1e-5, 1e-6, "FMA forward")
        # one fused multiply-add rounds once: never further than one ulp of the two-rounding product + sum
        assert_close(got, (t1.astype(np.float64) * t2 + t3).astype(np.float32), 2e-7, 1e-7, "FMA forward vs float64")
        init = rng.normal(0, 1, shape).astype(np.float32)
        for tid in range(3):
            want = oracle.backward_op(tid, OP.FMA, ug, t1, t2, t3, grad=init.copy())
            assert_close(run_bwd(ctx, tid, OP.FMA, ug, t1, t2, t3, grad_shape=shape, init=init), want, what="FMA d%d" % tid)
            assert_close(run_bwd(ctx, tid, OP.FMA, ug, t1, t2, t3, grad_shape=shape, init=init, accumulate=False),
                         oracle.backward_op(tid, OP.FMA, ug, t1, t2, t3), what="FMA d%d overwrite" % tid)


def test_pow_exponent_gradient(ctx):
    """POW.backward for the exponent (basics.mojo:359-376): the reference's known answers
    (test_backward.mojo:142-168) and seeded data with zeros in it (log(0) counts as 0)."""
    ones = np.ones((2, 3), np.float32)
    got = run_bwd(ctx, 1, OP.POW, ones, np.full((2, 3), 2, np.float32), grad_shape=(1,), exponent=2)
    assert_close(got, np.array([24 * np.log(2.0)], np.float32))
    got = run_bwd(ctx, 1, OP.POW, ones, np.zeros((2, 3), np.float32), grad_shape=(1,), exponent=0)
    assert_close(got, np.zeros(1, np.float32))
    rng = np.random.default_rng(13)
    for n, a in ((1000, 2.0), (70001, 3.0), (7, 1.0)):
        x = rng.uniform(0.1, 2.0, (n,)).astype(np.float32)
        x[::17] = 0.0
        ug = rng.normal(0, 1, (n,)).astype(np.float32)
        want = (np.where(x > 0, x.astype(np.float64) ** a * np.log(np.maximum(x, 1e-30).astype(np.float64)), 0.0) * ug).sum()
        init = np.array([0.25], np.float32)
        got = run_bwd(ctx, 1, OP.POW, ug, x, grad_shape=(1,), init=init, exponent=a)
        tol = 2e-5 * np.abs(np.where(x > 0, x.astype(np.float64) ** a * np.log(np.maximum(x, 1e-30)), 0.0) * ug).sum() + 1e-6
        assert abs(float(got[0]) - (want + 0.25)) <= tol, (n, a, got, want)
        ora = oracle.backward_op(1, OP.POW, ug, x, exponent=a, grad=init.copy())
        assert abs(float(got[0]) - float(ora[0])) <= 2 * tol      # the oracle sums serially in fp32
        got = run_bwd(ctx, 1, OP.POW, ug, x, grad_shape=(1,), init=init, accumulate=False, exponent=a)
        assert abs(float(got[0]) - want) <= tol


def test_relu_large_vectorised(ctx):
    rng = np.random.default_rng(3)
    x = rng.normal(0, 1, (8, 16, 28, 28)).astype(np.float32)
    ug = rng.normal(0, 1, x.shape).astype(np.float32)
    got = run_fwd(ctx, OP.RELU, x.shape, x)
    assert np.array_equal(got, np.maximum(x, 0) * (x > 0))
    assert np.array_equal(run_bwd(ctx, 0, OP.RELU, ug, x, grad_shape=x.shape), oracle.backward_op(0, OP.RELU, ug, x))


def test_copy_ops_and_fill(ctx):
    rng = np.random.default_rng(4)
    x = rng.normal(0, 1, (3, 32, 7, 7)).astype(np.float32)
    assert np.array_equal(run_fwd(ctx, OP.RESHAPE, (3, 1568), x).ravel(), x.ravel())
    assert np.array_equal(run_fwd(ctx, OP.FLATTEN, (3, 1568), x).ravel(), x.ravel())
    ug = rng.normal(0, 1, (3, 1568)).astype(np.float32)
    init = rng.normal(0, 1, x.shape).astype(np.float32)
    got = run_bwd(ctx, 0, OP.RESHAPE, ug, x, grad_shape=x.shape, init=init)
    assert_close(got.ravel(), init.ravel() + ug.ravel())
    d = ctx.empty((1001,))
    ctx._check(ctx.lib.mtl_fill_f32(ctx.handle, d.ptr, 1001, 2.5))
    assert np.array_equal(d.numpy(), np.full(1001, 2.5, np.float32))


# ------------------------------------------------------------------ reductions -----------------

RED = {"sum": OP.SUM, "mean": OP.MEAN, "max": OP.MAX}


def test_reductions(ctx):
    z = golden("ops")
    x = z["red__x"]
    for rname, op in RED.items():
        for axis in (None, 0, 1, 2):
            key = "red_%s_%s" % (rname, "all" if axis is None else axis)
            want = oracle.reduce_fwd(op, x, axis)
            assert_close(run_fwd(ctx, op, want.shape, x, axis=axis), want, 1e-5, 1e-5, key)
            ug = z[key + "__ug"]
            init = np.full(x.shape, 0.25, np.float32)
            want_g = oracle.reduce_bwd(op, ug, x, axis, grad=init.copy())
            assert_close(run_bwd(ctx, 0, op, ug, x, grad_shape=x.shape, init=init, axis=axis), want_g, 1e-5, 1e-6, key + " bwd")


def test_reduce_large_and_long_axis(ctx):
    rng = np.random.default_rng(5)
    x = rng.normal(0, 1, (300001,)).astype(np.float32)
    for op in (OP.SUM, OP.MEAN, OP.MAX):
        want = oracle.reduce_fwd(op, x)
        assert_close(run_fwd(ctx, op, (1,), x), want, 1e-4, 1e-3, "all %d" % op)  # summation order differs
    x = rng.normal(0, 1, (3, 2048, 5)).astype(np.float32)
    for op in (OP.SUM, OP.MAX):
        want = oracle.reduce_fwd(op, x, 1)
        assert_close(run_fwd(ctx, op, want.shape, x, axis=1), want, 1e-4, 1e-4, "long axis %d" % op)


def test_max_backward_ties(ctx):
    # test_backward.mojo:222-309
    t = np.ones((2, 3), np.float32)
    t[0, 0] = t[0, 1] = 2
    got = run_bwd(ctx, 0, OP.MAX, np.array([9], np.float32), t, grad_shape=t.shape)
    assert_close(got, oracle.backward_op(0, OP.MAX, np.array([9], np.float32), t))
    assert got[0, 0] == 4.5 and got[0, 1] == 4.5
    base = np.arange(1, 13, dtype=np.float32).reshape(2, 3, 2)
    for axis, first, ug_shape in ((0, 7, (1, 3, 2)), (1, 5, (2, 1, 2)), (2, 2, (2, 3, 1))):
        t = base.copy()
        t.ravel()[0] = first
        ug = np.full(ug_shape, 2, np.float32)
        assert_close(run_bwd(ctx, 0, OP.MAX, ug, t, grad_shape=t.shape, axis=axis), oracle.backward_op(0, OP.MAX, ug, t, axis=axis))


# ------------------------------------------------------------------ DOT ------------------------

def dot_all(ctx, a, b, ug):
    M, K = a.shape
    N = b.shape[1]
    c = run_fwd(ctx, OP.DOT, (M, N), a, b)
    da = run_bwd(ctx, 0, OP.DOT, ug, a, b, grad_shape=a.shape, accumulate=False)
    db = run_bwd(ctx, 1, OP.DOT, ug, a, b, grad_shape=b.shape, accumulate=False)
    return c, da, db


def test_dot_fp32_bit_exact(ctx):
    """MTL_MATH_FP32: ascending-k fmaf chains, identical bits to the reference's accumulation order."""
    z = golden("ops")
    ctx.set_math_mode(mb.MATH_FP32)
    try:
        for name in cases(z, "dot"):
            a, b, ug = z["dot%s__a" % name], z["dot%s__b" % name], z["dot%s__ug" % name]
            c, da, db = dot_all(ctx, a, b, ug)
            assert np.array_equal(c, oracle.dot(a, b)), name
            assert np.array_equal(da, oracle.dot_transpose_t2(ug, b)), name
            assert np.array_equal(db, oracle.dot_transpose_t1(a, ug)), name
            assert_close(c, z["dot%s__c" % name], 1e-5, 1e-5, "torch")
        # KAT: tests/mojo/test_ops.mojo:69-80 and test_backward.mojo:96-113
        c, da, db = dot_all(ctx, np.full((2, 3), 1, np.float32), np.full((3, 2), 2, np.float32), np.ones((2, 2), np.float32))
        assert np.all(c == 6) and np.all(da == 4) and np.all(db == 2)
    finally:
        ctx.set_math_mode(mb.MATH_TF32X3)


def rel_err(got, want):
    return float(np.max(np.abs(got.astype(np.float64) - want)) / np.max(np.abs(want)))


@pytest.mark.parametrize("M,K,N", [(128, 32, 128), (256, 96, 128), (384, 256, 256), (200, 136, 264), (512, 1024, 384)])
def test_dot_tensor_core(ctx, M, K, N):
    """tcgen05 path (all four operand major-ness combinations via fwd / dA / dB), both modes."""
    rng = np.random.default_rng(M + K + N)
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    b = rng.normal(0, 1, (K, N)).astype(np.float32)
    ug = rng.normal(0, 1, (M, N)).astype(np.float32)
    want = (a.astype(np.float64) @ b, ug.astype(np.float64) @ b.T.astype(np.float64), a.T.astype(np.float64) @ ug)
    for mode, tol in ((mb.MATH_TF32X3, 3e-5), (mb.MATH_TF32, 4e-3)):
        ctx.set_math_mode(mode)
        try:
            got = dot_all(ctx, a, b, ug)
        finally:
            ctx.set_math_mode(mb.MATH_TF32X3)
        assert ctx.device_status() == 0
        for g, w, what in zip(got, want, ("C", "dA", "dB")):
            e = rel_err(g, w)
            assert e < tol, "%s mode %d: normalised max error %.3e" % (what, mode, e)
    # element-wise tolerance of the 3xTF32 mode on unit-scale data: rtol 1e-4 / atol 1e-5
    a1 = rng.uniform(0, 1, (M, K)).astype(np.float32) / np.float32(K)
    b1 = rng.uniform(0, 1, (K, N)).astype(np.float32)
    assert_close(run_fwd(ctx, OP.DOT, (M, N), a1, b1), oracle.dot(a1, b1), 1e-4, 1e-5, "x3 elementwise")
    got_c = run_fwd(ctx, OP.DOT, (M, N), a, b)
    assert_close(got_c, want[0].astype(np.float32), 1e-4, 1e-5 * float(np.abs(want[0]).max()), "x3 elementwise, N(0,1) data")
    # accumulate into an existing gradient
    init = rng.normal(0, 1, (K, N)).astype(np.float32)
    got = run_bwd(ctx, 1, OP.DOT, ug, a, b, grad_shape=(K, N), init=init)
    assert rel_err(got, init + want[2]) < 3e-5


def test_dot_shapes_of_the_models(ctx):
    """Linear layers of the benchmark networks.  Tiny products run the ascending-k chain kernel
    (bit-exact); the thin N <= 16 products of the classifiers run the A-bandwidth-bound kernels,
    which re-associate the sum (compared at the reference's rtol = atol = 1e-5 scale)."""
    rng = np.random.default_rng(9)
    for M, K, N in ((32, 13, 1), (32, 1, 32), (32, 32, 32), (32, 32, 1), (64, 1568, 10), (16, 6272, 10),
                    (300, 1568, 10), (130, 6272, 10)):
        a = rng.normal(0, 1, (M, K)).astype(np.float32)
        b = (rng.normal(0, 1, (K, N)) / np.sqrt(K)).astype(np.float32)
        ug = rng.normal(0, 1, (M, N)).astype(np.float32)
        c, da, db = dot_all(ctx, a, b, ug)
        thin = M * K >= (1 << 16)
        if thin:
            assert_close(c, oracle.dot(a, b), 1e-5, 1e-5, "thin C %s" % ((M, K, N),))
            assert_close(db, oracle.dot_transpose_t1(a, ug), 1e-4, 1e-4, "thin dB %s" % ((M, K, N),))
        else:
            assert np.array_equal(c, oracle.dot(a, b))
            assert np.array_equal(db, oracle.dot_transpose_t1(a, ug))
        assert np.array_equal(da, oracle.dot_transpose_t2(ug, b))
        ctx.set_math_mode(mb.MATH_FP32)
        try:
            c, da, db = dot_all(ctx, a, b, ug)
        finally:
            ctx.set_math_mode(mb.MATH_TF32X3)
        assert np.array_equal(c, oracle.dot(a, b)) and np.array_equal(db, oracle.dot_transpose_t1(a, ug))


# ------------------------------------------------------------------ CONV2D ---------------------

def conv_all(ctx, x, w, b, ug, **kw):
    y = run_fwd(ctx, OP.CONV2D, ug.shape, x, w, b, **kw)
    bd = np.zeros_like(b)
    dx = run_bwd(ctx, 0, OP.CONV2D, ug, x, w, bd, grad_shape=x.shape, accumulate=False, **kw)
    dw = run_bwd(ctx, 1, OP.CONV2D, ug, x, w, bd, grad_shape=w.shape, accumulate=False, **kw)
    db = run_bwd(ctx, 2, OP.CONV2D, ug, x, w, bd, grad_shape=b.shape, accumulate=False, **kw)
    return y, dx, dw, db


def test_conv_reference_cases(ctx):
    """The padding / stride / dilation cases of tests/python/test_conv.mojo and the CNN layers."""
    z = golden("conv_pool")
    for name in cases(z, "conv_"):
        f = lambda k: z["conv_%s__%s" % (name, k)]
        a = f("attrs")
        kw = dict(padding=tuple(int(v) for v in a[0:2]), stride=tuple(int(v) for v in a[2:4]),
                  dilation=tuple(int(v) for v in a[4:6]))
        x, w, b, ug = f("x"), f("w"), f("b"), f("ug")
        y, dx, dw, db = conv_all(ctx, x, w, b, ug, **kw)
        assert y.shape == f("y").shape
        assert_close(y, oracle.conv2d_fwd(x, w, b, **kw), 1e-4, 1e-5, name + " y")
        assert_close(dx, oracle.conv2d_bwd(0, ug, x, w, **kw), 1e-4, 1e-4, name + " dx")
        assert_close(dw, oracle.conv2d_bwd(1, ug, x, w, **kw), 1e-4, 1e-3, name + " dw")
        assert_close(db, oracle.conv2d_bwd(2, ug, x, w, **kw), 1e-4, 1e-3, name + " db")
        assert_close(y, f("y"), 1e-4, 1e-5, name + " y (torch)")
        assert_close(dw, f("dw"), 1e-4, 1e-3, name + " dw (torch)")
        # accumulate semantics of backward_op (ops.mojo:498)
        init = np.full(w.shape, 0.5, np.float32)
        got = run_bwd(ctx, 1, OP.CONV2D, ug, x, w, np.zeros_like(b), grad_shape=w.shape, init=init, **kw)
        assert_close(got, init + oracle.conv2d_bwd(1, ug, x, w, **kw), 1e-4, 1e-3, name + " dw accumulate")


TC_CONV = [  # (N, C, H, W, K, R, S, pad): stride 1, dilation 1 -> implicit GEMM on tensor cores
    (4, 32, 8, 8, 64, 3, 3, 1),
    (6, 64, 14, 14, 128, 5, 5, 2),
    (3, 64, 12, 10, 64, 3, 3, 0),
    (5, 16, 14, 14, 32, 5, 5, 2),
    (2, 64, 56, 56, 64, 3, 3, 1),      # >= 4096 output pixels: the kernel gradient also runs on tensor cores
    (24, 64, 14, 14, 128, 5, 5, 2),    # conv2 of the widened CNN
    (40, 32, 12, 12, 48, 3, 3, 1),     # out-channels not a multiple of the tile, odd pixel boxes
    (9, 160, 10, 12, 40, 4, 5, 2),     # <= 64 output channels and a long reduction: two taps per instruction (forward)
]


@pytest.mark.parametrize("case", TC_CONV)
def test_conv_tensor_core(ctx, case):
    N, C, H, W, K, R, S, p = case
    rng = np.random.default_rng(sum(case))
    x = rng.normal(0, 1, (N, C, H, W)).astype(np.float32)
    w = (rng.normal(0, 1, (K, C, R, S)) / np.sqrt(C * R * S)).astype(np.float32)
    b = rng.normal(0, 1, K).astype(np.float32)
    kw = dict(padding=(p, p), stride=(1, 1), dilation=(1, 1))
    want_y = oracle.conv2d_fwd(x, w, b, **kw)
    ug = rng.normal(0, 1, want_y.shape).astype(np.float32)
    want = (want_y, oracle.conv2d_bwd(0, ug, x, w, **kw), oracle.conv2d_bwd(1, ug, x, w, **kw),
            oracle.conv2d_bwd(2, ug, x, w, **kw))
    for mode, tol in ((mb.MATH_TF32X3, 3e-5), (mb.MATH_TF32, 4e-3), (mb.MATH_FP32, 5e-6)):
        ctx.set_math_mode(mode)
        try:
            got = conv_all(ctx, x, w, b, ug, **kw)
        finally:
            ctx.set_math_mode(mb.MATH_TF32X3)
        assert ctx.device_status() == 0
        for g, wv, what in zip(got, want, ("y", "dx", "dw", "db")):
            e = rel_err(g, wv.astype(np.float64))
            assert e < tol, "%s mode %d: normalised max error %.3e" % (what, mode, e)
    # element-wise tolerance in 3xTF32 mode
    got = conv_all(ctx, x, w, b, ug, **kw)
    assert_close(got[0], want[0], 1e-4, 1e-5 * float(np.abs(want[0]).max()), "y x3 elementwise")
    init = rng.normal(0, 1, x.shape).astype(np.float32)
    acc = run_bwd(ctx, 0, OP.CONV2D, ug, x, w, np.zeros_like(b), grad_shape=x.shape, init=init, **kw)
    assert rel_err(acc, (init + want[1]).astype(np.float64)) < 3e-5


FIRST_LAYER_CONV = [  # few input channels, 28-pixel rows: the CUDA-core kernels written for conv1 of the CNNs
    (70, 1, 28, 28, 64, 5, 5, 2),
    (65, 3, 28, 28, 40, 3, 3, 1),
    (64, 1, 28, 28, 16, 5, 5, 2),
    (9, 1, 28, 28, 64, 5, 5, 2),       # batch below the threshold of the row-streaming kernel
]


@pytest.mark.parametrize("case", FIRST_LAYER_CONV)
def test_conv_first_layer(ctx, case):
    N, C, H, W, K, R, S, p = case
    rng = np.random.default_rng(sum(case))
    x = rng.normal(0, 1, (N, C, H, W)).astype(np.float32)
    w = (rng.normal(0, 1, (K, C, R, S)) / np.sqrt(C * R * S)).astype(np.float32)
    b = rng.normal(0, 1, K).astype(np.float32)
    kw = dict(padding=(p, p), stride=(1, 1), dilation=(1, 1))
    want_y = oracle.conv2d_fwd(x, w, b, **kw)
    ug = rng.normal(0, 1, want_y.shape).astype(np.float32)
    want = (want_y, oracle.conv2d_bwd(0, ug, x, w, **kw), oracle.conv2d_bwd(1, ug, x, w, **kw),
            oracle.conv2d_bwd(2, ug, x, w, **kw))
    got = conv_all(ctx, x, w, b, ug, **kw)
    for g, wv, what in zip(got, want, ("y", "dx", "dw", "db")):
        e = rel_err(g, wv.astype(np.float64))
        assert e < 1e-5, "%s: normalised max error %.3e" % (what, e)   # fp32 CUDA-core paths, re-associated sums
    init = rng.normal(0, 1, w.shape).astype(np.float32)
    acc = run_bwd(ctx, 1, OP.CONV2D, ug, x, w, np.zeros_like(b), grad_shape=w.shape, init=init, **kw)
    assert rel_err(acc, (init + want[2]).astype(np.float64)) < 1e-5


FUSED_CONV = [  # channel-major TC, pixel-major TC, first-layer rows kernel, generic CUDA-core kernel
    (6, 64, 14, 14, 128, 5, 5, 2), (5, 16, 14, 14, 32, 5, 5, 2), (70, 1, 28, 28, 64, 5, 5, 2), (3, 2, 9, 11, 5, 3, 3, 1),
]


@pytest.mark.parametrize("case", FUSED_CONV)
def test_conv_with_fused_relu_equals_two_calls(ctx, case):
    """mtl_conv2d_fwd_act == RELU.forward(CONV2D.forward(...)), bit for bit, on every kernel path."""
    N, C, H, W, K, R, S, p = case
    rng = np.random.default_rng(sum(case) + 1)
    x = ctx.array(rng.normal(0, 1, (N, C, H, W)).astype(np.float32))
    w = ctx.array((rng.normal(0, 1, (K, C, R, S)) / np.sqrt(C * R * S)).astype(np.float32))
    b = ctx.array(rng.normal(0, 1, K).astype(np.float32))
    kw = dict(padding=(p, p), stride=(1, 1), dilation=(1, 1))
    oh, ow = mb.conv2d_out_shape((N, C, H, W), (K, C, R, S), **kw)
    for mode in (mb.MATH_TF32X3, mb.MATH_TF32, mb.MATH_FP32):
        ctx.set_math_mode(mode)
        try:
            y = ctx.empty((N, K, oh, ow)); z = ctx.empty((N, K, oh, ow)); f = ctx.empty((N, K, oh, ow))
            ctx.forward_op(OP.CONV2D, y, x, w, b, **kw)
            ctx.forward_op(OP.RELU, z, y)
            ctx.forward_op(OP.CONV2D, f, x, w, b, fused_act=OP.RELU, **kw)
        finally:
            ctx.set_math_mode(mb.MATH_TF32X3)
        assert np.array_equal(f.numpy(), z.numpy()), "mode %d" % mode
        assert (z.numpy() == 0).any() and (z.numpy() > 0).any()


FUSED_CONV_POOL = [  # first-layer kernel that pools itself; odd shapes through scratch memory; tensor-core layers that
    # pool in the epilogue (row widths 14, 16, 12, 8 in registers, 10 through shared memory, partial channel tiles)
    (70, 1, 28, 28, 64, 5, 5, 2), (65, 3, 28, 28, 40, 3, 3, 1), (6, 64, 14, 14, 128, 5, 5, 2), (3, 2, 10, 12, 5, 3, 3, 1),
    (23, 32, 14, 14, 160, 3, 3, 1), (5, 32, 16, 16, 80, 3, 3, 1), (10, 16, 12, 12, 72, 3, 3, 1), (20, 16, 8, 8, 128, 3, 3, 1),
    (12, 16, 10, 10, 96, 3, 3, 1),
    # first layers that run on the tensor cores in plain TF32 mode: 3 input channels, two channel groups, 32-wide rows,
    # no padding, a ragged last tile
    (9, 3, 32, 32, 40, 3, 3, 1), (10, 1, 28, 28, 70, 3, 3, 1), (8, 1, 32, 32, 16, 5, 5, 2), (8, 1, 32, 32, 20, 5, 5, 0),
    (13, 1, 28, 28, 64, 5, 5, 2),
]


@pytest.mark.parametrize("case", FUSED_CONV_POOL)
def test_conv_relu_pool_equals_three_calls(ctx, case):
    """mtl_conv2d_fwd_act_pool == MAXPOOL2D.forward(RELU.forward(CONV2D.forward(...))): values and int32 indices."""
    import ctypes as Cc
    N, C, H, W, K, R, S, p = case
    rng = np.random.default_rng(sum(case) + 5)
    x = ctx.array(rng.normal(0, 1, (N, C, H, W)).astype(np.float32))
    w = ctx.array((rng.normal(0, 1, (K, C, R, S)) / np.sqrt(C * R * S)).astype(np.float32))
    b = ctx.array(rng.normal(0, 1, K).astype(np.float32))
    kw = dict(padding=(p, p), stride=(1, 1), dilation=(1, 1))
    oh, ow = mb.conv2d_out_shape((N, C, H, W), (K, C, R, S), **kw)
    pkw = dict(kernel_size=(2, 2), stride=(2, 2), padding=(0, 0), dilation=(1, 1))
    for mode in (mb.MATH_TF32X3, mb.MATH_TF32, mb.MATH_FP32):
        ctx.set_math_mode(mode)
        try:
            y, z = ctx.empty((N, K, oh, ow)), ctx.empty((N, K, oh, ow))
            want_v, want_i = ctx.empty((N, K, oh // 2, ow // 2)), ctx.empty((N, K, oh // 2, ow // 2), np.int32)
            ctx.forward_op(OP.CONV2D, y, x, w, b, **kw)
            ctx.forward_op(OP.RELU, z, y)
            ctx.forward_op(OP.MAXPOOL2D, want_v, z, indices=want_i, **pkw)
            got_v, got_i = ctx.empty((N, K, oh // 2, ow // 2)), ctx.empty((N, K, oh // 2, ow // 2), np.int32)
            d = mb.conv_desc(N, C, H, W, K, R, S, (p, p), (1, 1), (1, 1))
            pd = mb.conv_desc(N, K, oh, ow, 1, 2, 2, (0, 0), (2, 2), (1, 1))
            ctx._check(ctx.lib.mtl_conv2d_fwd_act_pool(ctx.handle, got_v.ptr, got_i.ptr, x.ptr, w.ptr, b.ptr, Cc.byref(d),
                                                       int(OP.RELU), Cc.byref(pd)))
        finally:
            ctx.set_math_mode(mb.MATH_TF32X3)
        if mode == mb.MATH_TF32 and C * R * S <= 32:
            # plain TF32: the fused first layer runs on the tensor cores, the three separate calls on
            # CUDA cores in fp32.  Values agree to TF32 accuracy; every argmax index lies in its window
            # and points at an activation that is the window's maximum to the same accuracy.
            zv, gv, gi = z.numpy(), got_v.numpy(), got_i.numpy()
            tol = 5e-3 * float(np.abs(zv).max())
            assert np.abs(gv - want_v.numpy()).max() <= tol, "values, TF32 first layer"
            ih, iw = gi // ow, gi % ow
            ph, pw = np.meshgrid(np.arange(oh // 2), np.arange(ow // 2), indexing="ij")
            assert np.array_equal(ih // 2, np.broadcast_to(ph, gi.shape)) and np.array_equal(iw // 2, np.broadcast_to(pw, gi.shape))
            picked = np.take_along_axis(zv.reshape(N, K, -1), gi.reshape(N, K, -1), axis=2).reshape(gv.shape)
            assert np.abs(picked - want_v.numpy()).max() <= tol, "argmax, TF32 first layer"
        else:
            assert np.array_equal(got_v.numpy(), want_v.numpy()), "values, mode %d" % mode
            assert np.array_equal(got_i.numpy(), want_i.numpy()), "indices, mode %d" % mode
        assert (got_v.numpy() == 0).any()


@pytest.mark.parametrize("case", [(70, 1, 28, 28, 64, 5, 5, 2), (10, 1, 28, 28, 70, 3, 3, 1), (9, 3, 32, 32, 40, 3, 3, 1),
                                  (8, 1, 32, 32, 20, 5, 5, 0), (37, 1, 28, 28, 64, 5, 5, 2)])
def test_first_layer_gradients_on_tensor_cores(ctx, case):
    """Plain TF32 mode: mtl_conv2d_bwd_pooled without dX on a first layer (C*R*S <= 31) rebuilds the dense
    gradient as a tensor-core operand and takes the bias gradient from a row of ones.  Compared with the
    fp32 CUDA-core result of the three reference-shaped calls, to TF32 accuracy."""
    import ctypes as Cc
    N, C, H, W, K, R, S, p = case
    rng = np.random.default_rng(sum(case) + 11)
    x = ctx.array(rng.normal(0, 1, (N, C, H, W)).astype(np.float32))
    w = ctx.array((rng.normal(0, 1, (K, C, R, S)) / np.sqrt(C * R * S)).astype(np.float32))
    b = ctx.array(rng.normal(0, 0.5, K).astype(np.float32))
    kw = dict(padding=(p, p), stride=(1, 1), dilation=(1, 1))
    pkw = dict(kernel_size=(2, 2), stride=(2, 2), padding=(0, 0), dilation=(1, 1))
    oh, ow = mb.conv2d_out_shape((N, C, H, W), (K, C, R, S), **kw)
    y, z = ctx.empty((N, K, oh, ow)), ctx.empty((N, K, oh, ow))
    pooled, idx = ctx.empty((N, K, oh // 2, ow // 2)), ctx.empty((N, K, oh // 2, ow // 2), np.int32)
    ctx.forward_op(OP.CONV2D, y, x, w, b, **kw)
    ctx.forward_op(OP.RELU, z, y)
    ctx.forward_op(OP.MAXPOOL2D, pooled, z, indices=idx, **pkw)
    pug = ctx.array(rng.normal(0, 1, (N, K, oh // 2, ow // 2)).astype(np.float32))
    g_z, g_y = ctx.empty((N, K, oh, ow)), ctx.empty((N, K, oh, ow))
    ctx.backward_op(0, OP.MAXPOOL2D, pug, z, grad=g_z, accumulate=False, indices=idx, **pkw)
    ctx.backward_op(0, OP.RELU, g_z, y, grad=g_y, accumulate=False)
    d = mb.conv_desc(N, C, H, W, K, R, S, (p, p), (1, 1), (1, 1))
    pd = mb.conv_desc(N, K, oh, ow, 1, 2, 2, (0, 0), (2, 2), (1, 1))
    for acc in (0, 1):
        init = [rng.normal(0, 1, s).astype(np.float32) for s in ((K, C, R, S), (K,))]
        want = [ctx.array(a) for a in init]
        for tid in (1, 2):
            ctx.backward_op(tid, OP.CONV2D, g_y, x, w, b, grad=want[tid - 1], accumulate=bool(acc), **kw)
        got = [ctx.array(a) for a in init]
        ctx.set_math_mode(mb.MATH_TF32)
        try:
            for act, pv in ((int(OP.RELU), pooled.ptr),):
                ctx._check(ctx.lib.mtl_conv2d_bwd_pooled(ctx.handle, None, got[0].ptr, got[1].ptr, pug.ptr, idx.ptr, pv,
                                                         x.ptr, None, w.ptr, Cc.byref(d), act, Cc.byref(pd), 0, acc, acc))
        finally:
            ctx.set_math_mode(mb.MATH_TF32X3)
        assert rel_err(got[0].numpy(), want[0].numpy().astype(np.float64)) < 4e-3, "dW acc %d" % acc
        assert rel_err(got[1].numpy(), want[1].numpy().astype(np.float64)) < 4e-3, "db acc %d" % acc
    assert ctx.device_status() == 0


@pytest.mark.parametrize("case", [(70, 1, 28, 28, 64, 5, 5, 2), (65, 3, 28, 28, 40, 3, 3, 1), (6, 2, 12, 12, 5, 3, 3, 1),
                                  (24, 64, 14, 14, 128, 5, 5, 2), (3, 64, 56, 56, 64, 3, 3, 1)])
def test_conv_backward_from_pooled_gradient(ctx, case):
    """mtl_conv2d_bwd_pooled == CONV2D.backward(RELU.backward(MAXPOOL2D.backward(ug))): the first-layer kernel
    that rebuilds the dense gradient in shared memory, the tensor-core path that scatters it into the
    channels-last operand copy, and the scratch-memory path."""
    import ctypes as Cc
    N, C, H, W, K, R, S, p = case
    rng = np.random.default_rng(sum(case) + 7)
    x = ctx.array(rng.normal(0, 1, (N, C, H, W)).astype(np.float32))
    w = ctx.array((rng.normal(0, 1, (K, C, R, S)) / np.sqrt(C * R * S)).astype(np.float32))
    b = ctx.array(rng.normal(0, 0.5, K).astype(np.float32))
    kw = dict(padding=(p, p), stride=(1, 1), dilation=(1, 1))
    pkw = dict(kernel_size=(2, 2), stride=(2, 2), padding=(0, 0), dilation=(1, 1))
    oh, ow = mb.conv2d_out_shape((N, C, H, W), (K, C, R, S), **kw)
    y, z = ctx.empty((N, K, oh, ow)), ctx.empty((N, K, oh, ow))
    pooled, idx = ctx.empty((N, K, oh // 2, ow // 2)), ctx.empty((N, K, oh // 2, ow // 2), np.int32)
    ctx.forward_op(OP.CONV2D, y, x, w, b, **kw)
    ctx.forward_op(OP.RELU, z, y)
    ctx.forward_op(OP.MAXPOOL2D, pooled, z, indices=idx, **pkw)
    pug = ctx.array(rng.normal(0, 1, (N, K, oh // 2, ow // 2)).astype(np.float32))
    # reference-shaped calls
    g_z, g_y = ctx.empty((N, K, oh, ow)), ctx.empty((N, K, oh, ow))
    ctx.backward_op(0, OP.MAXPOOL2D, pug, z, grad=g_z, accumulate=False, indices=idx, **pkw)
    ctx.backward_op(0, OP.RELU, g_z, y, grad=g_y, accumulate=False)
    d = mb.conv_desc(N, C, H, W, K, R, S, (p, p), (1, 1), (1, 1))
    pd = mb.conv_desc(N, K, oh, ow, 1, 2, 2, (0, 0), (2, 2), (1, 1))
    tc = C >= 16
    for mode in ((mb.MATH_TF32X3, mb.MATH_TF32) if tc else (mb.MATH_TF32X3,)):
        ctx.set_math_mode(mode)
        try:
            for acc in (0, 1):
                init = [rng.normal(0, 1, s).astype(np.float32) for s in ((N, C, H, W), (K, C, R, S), (K,))]
                want = [ctx.array(a) for a in init]
                for tid in range(3):
                    ctx.backward_op(tid, OP.CONV2D, g_y, x, w, b, grad=want[tid], accumulate=bool(acc), **kw)
                got = [ctx.array(a) for a in init]
                ctx._check(ctx.lib.mtl_conv2d_bwd_pooled(ctx.handle, got[0].ptr, got[1].ptr, got[2].ptr, pug.ptr, idx.ptr,
                                                         pooled.ptr, x.ptr, None, w.ptr, Cc.byref(d), int(OP.RELU),
                                                         Cc.byref(pd), acc, acc, acc))
                if tc:  # the same kernels on the same operand values: bitwise, bias sum within rounding
                    assert np.array_equal(got[0].numpy(), want[0].numpy()), "dX mode %d acc %d" % (mode, acc)
                    assert np.array_equal(got[1].numpy(), want[1].numpy()), "dW mode %d acc %d" % (mode, acc)
                else:
                    assert rel_err(got[0].numpy(), want[0].numpy().astype(np.float64)) < 1e-5
                    assert rel_err(got[1].numpy(), want[1].numpy().astype(np.float64)) < 1e-5
                assert rel_err(got[2].numpy(), want[2].numpy().astype(np.float64)) < 1e-5, "db acc %d" % acc
                # only the kernel and bias gradients (a first layer)
                part = [ctx.array(a) for a in init]
                ctx._check(ctx.lib.mtl_conv2d_bwd_pooled(ctx.handle, None, part[1].ptr, part[2].ptr, pug.ptr, idx.ptr,
                                                         pooled.ptr, x.ptr, None, w.ptr, Cc.byref(d), int(OP.RELU),
                                                         Cc.byref(pd), 0, acc, acc))
                assert rel_err(part[1].numpy(), want[1].numpy().astype(np.float64)) < (3e-5 if tc else 1e-5)
                assert rel_err(part[2].numpy(), want[2].numpy().astype(np.float64)) < 1e-5
                assert np.array_equal(part[0].numpy(), init[0])
        finally:
            ctx.set_math_mode(mb.MATH_TF32X3)
    assert ctx.device_status() == 0


FUSED_POOL = [  # (N, C, H, W, kernel, stride, pad): two-window float4, one-window float2, generic, overlapping
    (3, 4, 8, 8, 2, 2, 0), (3, 5, 14, 14, 2, 2, 0), (2, 3, 9, 9, 3, 2, 1), (2, 3, 8, 8, 3, 1, 1),
]


@pytest.mark.parametrize("case", FUSED_POOL)
def test_pool_backward_with_fused_relu_equals_two_calls(ctx, case):
    """mtl_maxpool2d_bwd_idx_act == RELU.backward(MAXPOOL2D.backward(...)) where the RELU feeds the pooling."""
    N, Cc, H, W, k, s, p = case
    rng = np.random.default_rng(sum(case) + 2)
    pre = rng.normal(0, 1, (N, Cc, H, W)).astype(np.float32)
    pre[0, 0, :4, :4] = -1.0                     # whole windows below zero: RELU output 0, mask 0
    kw = dict(kernel_size=(k, k), stride=(s, s), padding=(p, p), dilation=(1, 1))
    pre_d = ctx.array(pre)
    act = ctx.empty(pre.shape)
    ctx.forward_op(OP.RELU, act, pre_d)
    oh, ow = mb.conv2d_out_shape(pre.shape, (1, Cc, k, k), padding=(p, p), stride=(s, s))
    pooled, idx = ctx.empty((N, Cc, oh, ow)), ctx.empty((N, Cc, oh, ow), np.int32)
    ctx.forward_op(OP.MAXPOOL2D, pooled, act, indices=idx, **kw)
    ug = ctx.array(rng.normal(0, 1, (N, Cc, oh, ow)).astype(np.float32))
    for accumulate in (False, True):
        init = rng.normal(0, 1, pre.shape).astype(np.float32)
        # two calls: gradient of the RELU output, then of its input
        g_act = ctx.empty(pre.shape)
        ctx.backward_op(0, OP.MAXPOOL2D, ug, act, grad=g_act, accumulate=False, indices=idx, **kw)
        two = ctx.array(init)
        ctx.backward_op(0, OP.RELU, g_act, pre_d, grad=two, accumulate=accumulate)
        one = ctx.array(init)
        ctx.backward_op(0, OP.MAXPOOL2D, ug, act, grad=one, accumulate=accumulate, indices=idx, pooled=pooled,
                        fused_act=OP.RELU, **kw)
        if s >= k:
            assert np.array_equal(one.numpy(), two.numpy()), "accumulate=%s" % accumulate
        else:  # overlapping windows add with atomics: the order of the sum is not fixed
            assert_close(one.numpy(), two.numpy(), 1e-6, 1e-6, "accumulate=%s" % accumulate)


FUSED_BWD = [(6, 64, 14, 14, 128, 5, 5, 2), (2, 64, 56, 56, 64, 3, 3, 1), (70, 1, 28, 28, 64, 5, 5, 2),
             (5, 16, 14, 14, 32, 5, 5, 2), (3, 2, 9, 11, 5, 3, 3, 1)]


@pytest.mark.parametrize("case", FUSED_BWD)
def test_conv_backward_fused_equals_separate_calls(ctx, case):
    """mtl_conv2d_bwd_fused: dX and dW are the bits of the per-operand calls; db agrees within rounding."""
    N, C, H, W, K, R, S, p = case
    rng = np.random.default_rng(sum(case) + 3)
    x = ctx.array(rng.normal(0, 1, (N, C, H, W)).astype(np.float32))
    w = ctx.array((rng.normal(0, 1, (K, C, R, S)) / np.sqrt(C * R * S)).astype(np.float32))
    b = ctx.array(np.zeros(K, np.float32))
    kw = dict(padding=(p, p), stride=(1, 1), dilation=(1, 1))
    oh, ow = mb.conv2d_out_shape((N, C, H, W), (K, C, R, S), **kw)
    ug = ctx.array(rng.normal(0, 1, (N, K, oh, ow)).astype(np.float32))
    d = mb.conv_desc(N, C, H, W, K, R, S, (p, p), (1, 1), (1, 1))
    import ctypes as Cc
    for mode in (mb.MATH_TF32X3, mb.MATH_TF32):
        ctx.set_math_mode(mode)
        try:
            for acc in (0, 1):
                init = [rng.normal(0, 1, s).astype(np.float32) for s in ((N, C, H, W), (K, C, R, S), (K,))]
                sep = [ctx.array(a) for a in init]
                for tid in range(3):
                    ctx.backward_op(tid, OP.CONV2D, ug, x, w, b, grad=sep[tid], accumulate=bool(acc), **kw)
                fus = [ctx.array(a) for a in init]
                ctx._check(ctx.lib.mtl_conv2d_bwd_fused(ctx.handle, fus[0].ptr, fus[1].ptr, fus[2].ptr, ug.ptr, x.ptr, w.ptr,
                                                        Cc.byref(d), acc, acc, acc))
                assert np.array_equal(fus[0].numpy(), sep[0].numpy()), "dX mode %d acc %d" % (mode, acc)
                assert np.array_equal(fus[1].numpy(), sep[1].numpy()), "dW mode %d acc %d" % (mode, acc)
                assert rel_err(fus[2].numpy(), sep[2].numpy().astype(np.float64)) < 1e-5, "db"
                # a subset: only the kernel and bias gradients
                part = [ctx.array(a) for a in init]
                ctx._check(ctx.lib.mtl_conv2d_bwd_fused(ctx.handle, None, part[1].ptr, part[2].ptr, ug.ptr, x.ptr, w.ptr,
                                                        Cc.byref(d), 0, acc, acc))
                assert rel_err(part[1].numpy(), sep[1].numpy().astype(np.float64)) < 1e-5
                assert rel_err(part[2].numpy(), sep[2].numpy().astype(np.float64)) < 1e-5
                assert np.array_equal(part[0].numpy(), init[0])
        finally:
            ctx.set_math_mode(mb.MATH_TF32X3)
    assert ctx.device_status() == 0


# ------------------------------------------------------------------ MAXPOOL2D ------------------

def test_maxpool_reference_cases(ctx):
    z = golden("conv_pool")
    for name in cases(z, "pool_"):
        f = lambda k: z["pool_%s__%s" % (name, k)]
        a = [int(v) for v in f("attrs")]
        kw = dict(kernel_size=tuple(a[0:2]), padding=tuple(a[2:4]), stride=tuple(a[4:6]), dilation=tuple(a[6:8]))
        x, ug = f("x"), f("ug")
        want_y, want_idx = oracle.maxpool2d_fwd(x, return_indices=True, **kw)
        dx_d = ctx.array(x)
        y_d, idx_d = ctx.empty(want_y.shape), ctx.empty(want_y.shape, np.int32)
        ctx.forward_op(OP.MAXPOOL2D, y_d, dx_d, indices=idx_d, **kw)
        assert np.array_equal(y_d.numpy(), want_y), name          # bit-exact values
        assert np.array_equal(idx_d.numpy(), want_idx), name      # bit-exact argmax indices
        assert np.array_equal(idx_d.numpy(), f("idx")), name      # and the indices torch reports
        want_dx = oracle.maxpool2d_bwd(ug, x, **kw)
        got = run_bwd(ctx, 0, OP.MAXPOOL2D, ug, x, grad_shape=x.shape, accumulate=False, **kw)
        assert_close(got, want_dx, 1e-6, 1e-6, name + " dx (recompute)")
        g = ctx.zeros(x.shape)
        ctx.backward_op(0, OP.MAXPOOL2D, ctx.array(ug), dx_d, grad=g, indices=idx_d, accumulate=True, **kw)
        assert_close(g.numpy(), want_dx, 1e-6, 1e-6, name + " dx (indices)")
        assert_close(want_dx, f("dx"), 1e-6, 1e-6, name + " dx (torch)")


def test_maxpool_ties_nan_and_empty_windows(ctx):
    kw = dict(kernel_size=(2, 2), stride=(2, 2))
    x = np.ones((1, 1, 4, 4), np.float32)  # ties: the first element in (kx, ky) scan order wins
    y, idx = ctx.empty((1, 1, 2, 2)), ctx.empty((1, 1, 2, 2), np.int32)
    ctx.forward_op(OP.MAXPOOL2D, y, ctx.array(x), indices=idx, **kw)
    assert idx.numpy().ravel().tolist() == [0, 2, 8, 10]
    x[0, 0, 0, 0] = np.nan                # NaN never wins the strict `>` comparison
    x[0, 0, 2:, 2:] = -np.inf             # a window with nothing above -inf selects nothing
    ctx.forward_op(OP.MAXPOOL2D, y, ctx.array(x), indices=idx, **kw)
    want_y, want_idx = oracle.maxpool2d_fwd(x, return_indices=True, **kw)
    assert np.array_equal(idx.numpy(), want_idx) and idx.numpy().ravel()[0] == 1 and idx.numpy().ravel()[3] == -1
    assert np.array_equal(y.numpy(), want_y)
    ug = np.arange(1, 5, dtype=np.float32).reshape(1, 1, 2, 2)
    got = run_bwd(ctx, 0, OP.MAXPOOL2D, ug, x, grad_shape=x.shape, accumulate=False, **kw)
    assert np.array_equal(got, oracle.maxpool2d_bwd(ug, x, **kw))  # the empty window routes nothing


def test_maxpool_overlapping_windows_accumulate(ctx):
    rng = np.random.default_rng(11)
    x = rng.normal(0, 1, (2, 3, 9, 11)).astype(np.float32)
    kw = dict(kernel_size=(3, 3), stride=(1, 2), padding=(1, 1))
    want_y = oracle.maxpool2d_fwd(x, **kw)
    ug = rng.normal(0, 1, want_y.shape).astype(np.float32)
    init = rng.normal(0, 1, x.shape).astype(np.float32)
    got = run_bwd(ctx, 0, OP.MAXPOOL2D, ug, x, grad_shape=x.shape, init=init, **kw)
    assert_close(got, init + oracle.maxpool2d_bwd(ug, x, **kw), 1e-5, 1e-5)


# ------------------------------------------------------------------ Adam -----------------------

def test_adam_matches_oracle(ctx):
    rng = np.random.default_rng(12)
    n = 28938 + 3  # the CNN's parameter count plus an unaligned tail
    p = rng.normal(0, 1, n).astype(np.float32)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    dp, dm, dv = ctx.array(p), ctx.array(m), ctx.array(v)
    for t in range(1, 6):
        g = rng.normal(0, 0.1, n).astype(np.float32)
        oracle.adam_step(p, g, m, v, 1e-3, 0.9, 0.999, 1e-8, t)
        ctx.adam_step(dp, ctx.array(g), dm, dv, n, 1e-3, 0.9, 0.999, 1e-8, t)
        assert_close(dp.numpy(), p, 1e-5, 1e-6, "params step %d" % t)
        assert_close(dm.numpy(), m, 1e-5, 1e-7, "m step %d" % t)
        assert_close(dv.numpy(), v, 1e-5, 1e-9, "v step %d" % t)


# ------------------------------------------------------------------ error behaviour ------------

def test_invalid_arguments_return_status(ctx):
    L, h = ctx.lib, ctx.handle
    a = ctx.zeros((4, 4))
    assert L.mtl_dot_fwd(h, a.ptr, a.ptr, None, 4, 4, 4) == 1
    assert L.mtl_unary_fwd(h, OP.DOT, a.ptr, a.ptr, 16, 0.0, 0.0) == 1
    assert b"not a unary" in L.mtl_last_error(h)
    assert L.mtl_adam_step(h, a.ptr, a.ptr, a.ptr, a.ptr, 16, 1e-3, 0.9, 0.999, 1e-8, 0, 1.0) == 1
    s2 = (2 * np.ones(1)).astype(np.int64)
    with pytest.raises(mb.MantleError):
        ctx.forward_op(OP.ADD, a, ctx.zeros((3,)), ctx.zeros((4,)))
    with pytest.raises(mb.MantleError):
        ctx.forward_op(25, a, a)  # SLICE
    assert ctx.device_status() == 0
    assert ctx.launch_count() > 0


def test_channels_last_twins(ctx):
    """mtl_conv2d_fwd_act_pool_cl writes a channels-last copy of the pooled output (from the first-layer
    kernel and from the extra-pass path); consumers given that copy as X_cl produce the bits they produce
    from X alone (plain TF32 mode) and ignore it in 3xTF32 mode."""
    import ctypes as Cc
    rng = np.random.default_rng(91)
    for (N, C, H, W, K, R, S, p) in ((70, 1, 28, 28, 64, 5, 5, 2), (6, 8, 12, 12, 16, 3, 3, 1)):
        x = ctx.array(rng.normal(0, 1, (N, C, H, W)).astype(np.float32))
        w = ctx.array((rng.normal(0, 1, (K, C, R, S)) / np.sqrt(C * R * S)).astype(np.float32))
        b = ctx.array(rng.normal(0, 1, K).astype(np.float32))
        d = mb.conv_desc(N, C, H, W, K, R, S, (p, p), (1, 1), (1, 1))
        pd = mb.conv_desc(N, K, H, W, 1, 2, 2, (0, 0), (2, 2), (1, 1))
        pooled, idx, twin = ctx.empty((N, K, H // 2, W // 2)), ctx.empty((N, K, H // 2, W // 2), np.int32), ctx.empty((N, H // 2, W // 2, K))
        ctx._check(ctx.lib.mtl_conv2d_fwd_act_pool_cl(ctx.handle, pooled.ptr, idx.ptr, twin.ptr, x.ptr, None, w.ptr, b.ptr,
                                                      Cc.byref(d), int(OP.RELU), Cc.byref(pd)))
        assert np.array_equal(twin.numpy(), pooled.numpy().transpose(0, 2, 3, 1))
    # consumer: the widened CNN's second layer
    N, C, H, W, K = 12, 64, 14, 14, 128
    x_h = rng.normal(0, 1, (N, C, H, W)).astype(np.float32)
    x, x_cl = ctx.array(x_h), ctx.array(np.ascontiguousarray(x_h.transpose(0, 2, 3, 1)))
    w = ctx.array((rng.normal(0, 1, (K, C, 5, 5)) / 40.0).astype(np.float32))
    b = ctx.array(rng.normal(0, 1, K).astype(np.float32))
    ug = ctx.array(rng.normal(0, 1, (N, K, H, W)).astype(np.float32))
    d = mb.conv_desc(N, C, H, W, K, 5, 5, (2, 2), (1, 1), (1, 1))
    pd = mb.conv_desc(N, K, H, W, 1, 2, 2, (0, 0), (2, 2), (1, 1))
    for mode in (mb.MATH_TF32, mb.MATH_TF32X3):
        ctx.set_math_mode(mode)
        try:
            outs = []
            for cl in (None, x_cl.ptr):
                pooled, idx = ctx.empty((N, K, 7, 7)), ctx.empty((N, K, 7, 7), np.int32)
                ctx._check(ctx.lib.mtl_conv2d_fwd_act_pool_cl(ctx.handle, pooled.ptr, idx.ptr, None, x.ptr, cl, w.ptr, b.ptr,
                                                              Cc.byref(d), int(OP.RELU), Cc.byref(pd)))
                dx, dw, db = ctx.empty((N, C, H, W)), ctx.empty((K, C, 5, 5)), ctx.empty((K,))
                ctx._check(ctx.lib.mtl_conv2d_bwd_fused_cl(ctx.handle, dx.ptr, dw.ptr, db.ptr, ug.ptr, x.ptr, cl, w.ptr,
                                                           Cc.byref(d), 0, 0, 0))
                outs.append([a.numpy() for a in (pooled, idx, dx, dw, db)])
        finally:
            ctx.set_math_mode(mb.MATH_TF32X3)
        for a, b_ in zip(*outs):
            assert np.array_equal(a, b_), "mode %d" % mode
    assert ctx.device_status() == 0


@pytest.mark.parametrize("B,C", [(37, 10), (2048, 10), (5, 3), (300, 130)])
def test_cross_entropy_equals_nine_operator_calls(ctx, B, C):
    """mtl_cross_entropy_fwd / _bwd == the reference's CrossEntropyLoss graph run node by node (loss.mojo:45-61,
    activations.mojo:94-108), forward value and logits gradient, ties in the row maximum included."""
    rng = np.random.default_rng(B * 131 + C)
    xh = rng.normal(0, 2, (B, C)).astype(np.float32)
    xh[0, :] = 0.5                       # a row of ties: MAX.backward splits evenly
    xh[1, 0] = xh[1, 1] = xh[1].max() + 1
    yh = np.eye(C, dtype=np.float32)[rng.integers(0, C, B)]
    yh[2] = rng.uniform(0, 1, C)         # soft targets
    x, y = ctx.array(xh), ctx.array(yh)
    scale = np.float32(-1.0 / B)
    mx, sm, lg = ctx.empty((B, 1)), ctx.empty((B, 1)), ctx.empty((B, 1))
    xm, ex, ls, t = ctx.empty((B, C)), ctx.empty((B, C)), ctx.empty((B, C)), ctx.empty((B, C))
    ret, loss, lit = ctx.empty((1,)), ctx.empty((1,)), ctx.array(np.array([scale], np.float32))
    ctx.forward_op(OP.MAX, mx, x, axis=1)
    ctx.forward_op(OP.SUB, xm, x, mx)
    ctx.forward_op(OP.EXP, ex, xm)
    ctx.forward_op(OP.SUM, sm, ex, axis=1)
    ctx.forward_op(OP.LOG, lg, sm)
    ctx.forward_op(OP.SUB, ls, xm, lg)
    ctx.forward_op(OP.MUL, t, y, ls)
    ctx.forward_op(OP.SUM, ret, t)
    ctx.forward_op(OP.MUL, loss, ret, lit)
    # backward, node by node in reverse, every gradient buffer starting at zero
    g = {k: ctx.zeros(s) for k, s in (("loss", (1,)), ("ret", (1,)), ("t", (B, C)), ("ls", (B, C)), ("xm", (B, C)),
                                      ("lg", (B, 1)), ("sm", (B, 1)), ("ex", (B, C)), ("mx", (B, 1)), ("x", (B, C)))}
    ctx._check(ctx.lib.mtl_fill_f32(ctx.handle, g["loss"].ptr, 1, 1.0))
    ctx.backward_op(0, OP.MUL, g["loss"], ret, lit, grad=g["ret"])
    ctx.backward_op(0, OP.SUM, g["ret"], t, grad=g["t"])
    ctx.backward_op(1, OP.MUL, g["t"], y, ls, grad=g["ls"])
    ctx.backward_op(0, OP.SUB, g["ls"], xm, lg, grad=g["xm"])
    ctx.backward_op(1, OP.SUB, g["ls"], xm, lg, grad=g["lg"])
    ctx.backward_op(0, OP.LOG, g["lg"], sm, grad=g["sm"])
    ctx.backward_op(0, OP.SUM, g["sm"], ex, grad=g["ex"], axis=1)
    ctx.backward_op(0, OP.EXP, g["ex"], xm, grad=g["xm"])
    ctx.backward_op(0, OP.SUB, g["xm"], x, mx, grad=g["x"])
    ctx.backward_op(1, OP.SUB, g["xm"], x, mx, grad=g["mx"])
    ctx.backward_op(0, OP.MAX, g["mx"], x, grad=g["x"], axis=1)
    got_loss = ctx.empty((1,))
    ctx._check(ctx.lib.mtl_cross_entropy_fwd(ctx.handle, got_loss.ptr, x.ptr, y.ptr, B, C, float(scale)))
    assert_close(got_loss.numpy(), loss.numpy(), 2e-6, 1e-7, "loss")
    want_loss = -np.sum(yh.astype(np.float64) * (xh - xh.max(1, keepdims=True) -
                                                 np.log(np.exp(xh.astype(np.float64) - xh.max(1, keepdims=True)).sum(1, keepdims=True)))) / B
    assert abs(float(got_loss.numpy()[0]) - want_loss) <= 1e-5 * abs(want_loss)
    for acc in (0, 1):
        init = rng.normal(0, 1, (B, C)).astype(np.float32)
        got = ctx.array(init)
        ctx._check(ctx.lib.mtl_cross_entropy_bwd(ctx.handle, got.ptr, x.ptr, y.ptr, B, C, float(scale), acc))
        want = g["x"].numpy() + (init if acc else 0)
        assert_close(got.numpy(), want, 1e-5, 1e-7 * float(np.abs(g["x"].numpy()).max()) + 1e-9, "dlogits acc %d" % acc)
    # both in one launch: the same bits as the two calls
    sep_loss, sep_grad = got_loss.numpy(), ctx.empty((B, C))
    ctx._check(ctx.lib.mtl_cross_entropy_bwd(ctx.handle, sep_grad.ptr, x.ptr, y.ptr, B, C, float(scale), 0))
    one_loss, one_grad = ctx.empty((1,)), ctx.array(rng.normal(0, 1, (B, C)).astype(np.float32))
    ctx._check(ctx.lib.mtl_cross_entropy_fwd_grad(ctx.handle, one_loss.ptr, one_grad.ptr, x.ptr, y.ptr, B, C, float(scale)))
    assert np.array_equal(one_loss.numpy(), sep_loss) and np.array_equal(one_grad.numpy(), sep_grad.numpy())
    assert ctx.device_status() == 0


def test_one_hot_on_device(ctx):
    """mtl_one_hot_f32 == the host loop of examples/mnist.mojo:92-97 (fp32 labels, Int() truncation)."""
    rng = np.random.default_rng(77)
    for B, C in ((2048, 10), (37, 3), (5, 1)):
        lab = rng.integers(0, C, B).astype(np.float32)
        lab[0] = C - 1 + 0.75 if C > 1 else 0.25      # truncates to a valid class
        want = oracle.one_hot(lab, C)
        assert np.array_equal(want, np.eye(C, dtype=np.float32)[lab.astype(np.int64)])
        d_lab, out = ctx.array(lab), ctx.empty((B, C))
        ctx._check(ctx.lib.mtl_one_hot_f32(ctx.handle, out.ptr, d_lab.ptr, B, C))
        assert np.array_equal(out.numpy(), want)
    lab = np.array([0, 5, -3, 2], np.float32)            # 5 and -3 are outside [0, 3): zero rows
    out = ctx.empty((4, 3))
    ctx._check(ctx.lib.mtl_one_hot_f32(ctx.handle, out.ptr, ctx.array(lab).ptr, 4, 3))
    assert np.array_equal(out.numpy(), oracle.one_hot(lab, 3)) and out.numpy()[1].sum() == 0 and out.numpy()[2].sum() == 0


def test_bounded_wait_runs_out_and_the_context_stays_usable(ctx):
    """A device-side wait that can never complete gives up after its budget (1 ms here), the kernel
    reports MTL_ERR_TIMEOUT through the context's status word and returns; the next operator works
    and the status reads clean again.  Nothing faults or hangs: the wait is the same bounded wait all
    tensor-core kernels use (with a 4 s budget that a correct run never reaches)."""
    import ctypes as C
    assert ctx.device_status() == 0
    waited = C.c_int32()
    ctx._check(ctx.lib.mtl_selftest_bounded_wait(ctx.handle, 1000, C.byref(waited)))
    assert 900 <= waited.value < 100000, "waited %d us for a 1000 us budget" % waited.value
    assert ctx.device_status() == 5          # MTL_ERR_TIMEOUT, read and cleared
    assert ctx.device_status() == 0
    rng = np.random.default_rng(77)
    a = rng.normal(0, 1, (256, 128)).astype(np.float32)
    b = rng.normal(0, 1, (128, 256)).astype(np.float32)
    got = run_fwd(ctx, OP.DOT, (256, 256), a, b)
    assert rel_err(got, a.astype(np.float64) @ b) < 3e-5
    assert ctx.device_status() == 0
    assert ctx.lib.mtl_selftest_bounded_wait(ctx.handle, 0, None) == 1     # MTL_ERR_INVALID


@pytest.mark.parametrize("M,K,N", [(256, 6272, 10), (2048, 6272, 10), (64, 1568, 10), (37, 515, 3), (300, 130, 16), (8, 40, 1),
                                   (37, 516, 3), (300, 132, 16), (5, 2052, 7), (1000, 1024, 12), (19, 4, 5)])
def test_linear_layer_as_one_call_each_way(ctx, M, K, N):
    """mtl_linear_fwd / mtl_linear_bwd against the reference's operator sequence on the oracle (DOT then ADD
    of the bias; DOT.backward for both operands, ADD.backward with un-broadcasting for the bias) and
    against the separate entry points of this library, in both accumulate settings."""
    import ctypes as C
    rng = np.random.default_rng(M * 7 + K + N)
    a = rng.normal(0, 1, (M, K)).astype(np.float32)
    w = (rng.normal(0, 1, (K, N)) / np.sqrt(K)).astype(np.float32)
    b = rng.normal(0, 1, (N,)).astype(np.float32)
    ug = rng.normal(0, 1, (M, N)).astype(np.float32)
    L, h = ctx.lib, ctx.handle
    da_, dw_, db_, dug = ctx.array(a), ctx.array(w), ctx.array(b), ctx.array(ug)
    c = ctx.empty((M, N))
    ctx._check(L.mtl_linear_fwd(h, c.ptr, da_.ptr, dw_.ptr, db_.ptr, M, K, N))
    want = oracle.binary_fwd(OP.ADD, oracle.dot(a, w), b)
    assert_close(c.numpy(), want, 1e-5, 1e-5, "Linear forward")
    ctx._check(L.mtl_linear_fwd(h, c.ptr, da_.ptr, dw_.ptr, None, M, K, N))       # no bias: plain DOT
    assert_close(c.numpy(), oracle.dot(a, w), 1e-5, 1e-5, "Linear forward without bias")
    want_da, want_dw = oracle.dot_transpose_t2(ug, w), oracle.dot_transpose_t1(a, ug)
    want_db = oracle.binary_bwd(OP.ADD, 1, ug, want, b)
    for acc in (0, 1):
        ia, iw, ib = (rng.normal(0, 1, s).astype(np.float32) for s in ((M, K), (K, N), (N,)))
        ga, gw, gb = ctx.array(ia), ctx.array(iw), ctx.array(ib)
        ctx._check(L.mtl_linear_bwd(h, ga.ptr, gw.ptr, gb.ptr, dug.ptr, da_.ptr, dw_.ptr, M, K, N, acc, acc, acc))
        assert_close(ga.numpy(), want_da + acc * ia, 1e-5, 1e-5, "dA acc=%d" % acc)
        assert_close(gw.numpy(), want_dw + acc * iw, 1e-4, 1e-4, "dB acc=%d" % acc)     # sums over the batch, re-associated
        assert_close(gb.numpy(), want_db + acc * ib, 1e-4, 1e-4, "dbias acc=%d" % acc)
    # any subset of the three gradients
    gw2 = ctx.zeros((K, N))
    ctx._check(L.mtl_linear_bwd(h, None, gw2.ptr, None, dug.ptr, da_.ptr, None, M, K, N, 0, 0, 0))
    assert np.array_equal(gw2.numpy(), gw.numpy() - iw) or np.allclose(gw2.numpy(), want_dw, 1e-4, 1e-4)
    # two calls in a row give identical bits (the ticket counters are back at zero, the fold order is fixed)
    gw3 = ctx.zeros((K, N))
    ctx._check(L.mtl_linear_bwd(h, None, gw3.ptr, None, dug.ptr, da_.ptr, None, M, K, N, 0, 0, 0))
    assert np.array_equal(gw2.numpy(), gw3.numpy())
    c2 = ctx.empty((M, N))
    ctx._check(L.mtl_linear_fwd(h, c2.ptr, da_.ptr, dw_.ptr, None, M, K, N))
    assert np.array_equal(c.numpy(), c2.numpy())
    # MTL_MATH_FP32 keeps the reference's ascending chain bit for bit (separate operator kernels)
    ctx.set_math_mode(mb.MATH_FP32)
    try:
        ctx._check(L.mtl_linear_fwd(h, c.ptr, da_.ptr, dw_.ptr, None, M, K, N))
        assert np.array_equal(c.numpy(), oracle.dot(a, w))
    finally:
        ctx.set_math_mode(mb.MATH_TF32X3)
    assert ctx.device_status() == 0
