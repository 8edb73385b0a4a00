"""TRANSPOSE / SLICE / CONCAT / SPLIT: the CPU restatement against the reference's known answers
(tests/mojo/test_ops.mojo:199-228, tests/mojo/test_mlops.mojo:356-760, tests/mojo/test_dynamic_ops.mojo) and
the strided-copy kernels against the restatement, bit for bit."""
import ctypes as C

import numpy as np
import pytest

import oracle
from oracle import layout


def iota(*shape):
    return np.arange(int(np.prod(shape)), dtype=np.float32).reshape(shape)


# ---------------------------------------------------------------- oracle vs the reference's KATs

def test_transpose_known_answers():
    t = iota(2, 3, 4)
    # test_ops.mojo:199-215: reversed axes -> (4, 3, 2) with expected[k, j, i] = t[i, j, k]
    got = layout.transpose_fwd(t)
    assert got.shape == (4, 3, 2) and all(got[k, j, i] == t[i, j, k] for i in range(2) for j in range(3) for k in range(4))
    # test_ops.mojo:217-228: axes (1, 2, 0) -> (3, 4, 2) with expected[j, k, i] = t[i, j, k]
    got = layout.transpose_fwd(t, (1, 2, 0))
    assert got.shape == (3, 4, 2) and all(got[j, k, i] == t[i, j, k] for i in range(2) for j in range(3) for k in range(4))
    assert np.array_equal(layout.transpose_bwd(got, t.shape, (1, 2, 0)), t)


def test_slice_known_answers():
    t = iota(3, 4, 5)
    # test_mlops.mojo:356-422: Slice(1, 3, 1) on each axis
    for ax, want in ((0, t[1:3]), (1, t[:, 1:3]), (2, t[:, :, 1:3])):
        assert np.array_equal(layout.slice_fwd(t, [1], [3], [1], [ax]), want)
    # :425-502 Slice(1, 6, 2) and :504-581 Slice(6, 1, -2): rows 1, 3, 5 and 6, 4, 2
    for shape, ax in (((10, 2, 2), 0), ((2, 10, 2), 1), ((2, 2, 10), 2)):
        t = iota(*shape)
        assert np.array_equal(layout.slice_fwd(t, [1], [6], [2], [ax]), np.take(t, [1, 3, 5], axis=ax))
        assert np.array_equal(layout.slice_fwd(t, [6], [1], [-2], [ax]), np.take(t, [6, 4, 2], axis=ax))
    # :583-673 several axes at once; a negative start / end pair counts from the end (-43, -30 of 50 -> 7..19)
    t = iota(20, 32, 40)
    got = layout.slice_fwd(t, [1, 3, 5], [6, 10, 15], [2, 3, 2])
    assert got.shape == (3, 3, 5) and got[2, 1, 4] == 5 * 32 * 40 + 6 * 40 + 13
    t = iota(6, 8, 10, 50)
    got = layout.slice_fwd(t, [1, 3, 5, -43], [6, 8, 9, -30], [2, 3, 2, 4])
    assert got.shape == (3, 2, 2, 4) and np.array_equal(got[0, 0, 0], t[1, 3, 5, [7, 11, 15, 19]])
    # :676-760 backward: ones land on the sliced positions of a zero tensor
    res = layout.slice_bwd(np.ones((2, 3, 2), np.float32), (2, 10, 2), [1], [6], [2], [1])
    want = np.zeros((2, 10, 2), np.float32)
    want[:, [1, 3, 5]] = 1
    assert np.array_equal(res, want)


def test_concat_split_known_answers():
    # test_dynamic_ops.mojo: three tensors joined along axis 0, 1 and 2; SPLIT with sections is the inverse
    a, b, c = iota(2, 3, 4), iota(2, 3, 4) + 100, iota(2, 3, 4) + 200
    for dim in (0, 1, 2):
        got = layout.concat_fwd([a, b, c], dim)
        assert np.array_equal(got, np.concatenate([a, b, c], axis=dim))
        for j, t in enumerate((a, b, c)):
            assert np.array_equal(layout.concat_bwd(got, [a.shape, b.shape, c.shape], j, dim), t)
    t = iota(4, 12, 3)
    parts = layout.split_fwd(t, [5, 5, 2], 1)
    assert [p.shape for p in parts] == [(4, 5, 3), (4, 5, 3), (4, 2, 3)]
    assert np.array_equal(parts[2], t[:, 10:12])
    assert np.array_equal(layout.split_bwd(parts, t.shape, [5, 5, 2], 1), t)


# ---------------------------------------------------------------- kernels vs the oracle

def _shape(s):
    return (C.c_int64 * len(s))(*s)


@pytest.mark.gpu
def test_transpose_and_slice_kernels(ctx):
    import mantle_b200 as mb
    L, h = ctx.lib, ctx.handle
    rng = np.random.default_rng(5)
    for shape, axes in (((2, 3, 4), None), ((2, 3, 4), (1, 2, 0)), ((5, 1, 7, 3), (3, 0, 2, 1)), ((64, 33), None),
                        ((3, 4, 5, 2, 3), (4, 2, 0, 3, 1))):
        t = rng.normal(0, 1, shape).astype(np.float32)
        want = layout.transpose_fwd(t, axes)
        out = ctx.empty(want.shape)
        ax = None if axes is None else (C.c_int32 * len(axes))(*axes)
        ctx._check(L.mtl_transpose_fwd(h, out.ptr, ctx.array(t).ptr, len(shape), _shape(shape), ax))
        assert np.array_equal(out.numpy(), want)
        ug = rng.normal(0, 1, want.shape).astype(np.float32)
        init = rng.normal(0, 1, shape).astype(np.float32)
        for acc in (0, 1):
            g = ctx.array(init)
            ctx._check(L.mtl_transpose_bwd(h, g.ptr, ctx.array(ug).ptr, len(shape), _shape(shape), ax, acc))
            assert np.array_equal(g.numpy(), layout.transpose_bwd(ug, shape, axes) + (init if acc else 0))
    cases = [((3, 4, 5), [1], [3], [1], [0]), ((3, 4, 5), [1], [3], [1], [2]), ((10, 2, 2), [1], [6], [2], [0]),
             ((2, 10, 2), [6], [1], [-2], [1]), ((20, 32, 40), [1, 3, 5], [6, 10, 15], [2, 3, 2], None),
             ((6, 8, 10, 50), [1, 3, 5, -43], [6, 8, 9, -30], [2, 3, 2, 4], None), ((7, 9), [-3], [9], [1], [1])]
    for shape, st, en, sp, ax in cases:
        t = rng.normal(0, 1, shape).astype(np.float32)
        want = layout.slice_fwd(t, st, en, sp, ax)
        d = mb.slice_desc(st, en, sp, ax)
        oshape = (C.c_int64 * len(shape))()
        assert L.mtl_slice_out_shape(len(shape), _shape(shape), C.byref(d), oshape) == 0
        assert tuple(oshape) == want.shape
        out = ctx.empty(want.shape)
        ctx._check(L.mtl_slice_fwd(h, out.ptr, ctx.array(t).ptr, len(shape), _shape(shape), C.byref(d)))
        assert np.array_equal(out.numpy(), want)
        ug = rng.normal(0, 1, want.shape).astype(np.float32)
        init = rng.normal(0, 1, shape).astype(np.float32)
        for acc in (0, 1):
            g = ctx.array(init)
            ctx._check(L.mtl_slice_bwd(h, g.ptr, ctx.array(ug).ptr, len(shape), _shape(shape), C.byref(d), acc))
            assert np.array_equal(g.numpy(), layout.slice_bwd(ug, shape, st, en, sp, ax) + (init if acc else 0))
    # refused: an empty slice, a zero step, an index outside the axis
    t = ctx.array(np.zeros((4, 4), np.float32))
    out = ctx.empty((4, 4))
    for d in (mb.slice_desc([3], [1], [1], [0]), mb.slice_desc([0], [2], [0], [0]), mb.slice_desc([4], [0], [-1], [0])):
        assert L.mtl_slice_fwd(h, out.ptr, t.ptr, 2, _shape((4, 4)), C.byref(d)) != 0


@pytest.mark.gpu
def test_concat_and_split_kernels(ctx):
    L, h = ctx.lib, ctx.handle
    rng = np.random.default_rng(6)
    for shapes, dim in ((((2, 3, 4), (5, 3, 4), (1, 3, 4)), 0), (((2, 3, 4), (2, 6, 4)), 1), (((2, 3, 4), (2, 3, 1), (2, 3, 7)), 2)):
        ts = [rng.normal(0, 1, s).astype(np.float32) for s in shapes]
        want = layout.concat_fwd(ts, dim)
        dev = [ctx.array(t) for t in ts]
        ptrs = (C.c_void_p * len(ts))(*[a.ptr.value if hasattr(a.ptr, "value") else a.ptr for a in dev])
        flat = (C.c_int64 * (len(ts) * 3))(*[v for s in shapes for v in s])
        out = ctx.empty(want.shape)
        ctx._check(L.mtl_concat_fwd(h, out.ptr, ptrs, len(ts), 3, flat, dim))
        assert np.array_equal(out.numpy(), want)
        ug = rng.normal(0, 1, want.shape).astype(np.float32)
        for j, s in enumerate(shapes):
            init = rng.normal(0, 1, s).astype(np.float32)
            for acc in (0, 1):
                g = ctx.array(init)
                ctx._check(L.mtl_concat_bwd(h, g.ptr, ctx.array(ug).ptr, j, len(ts), 3, flat, dim, acc))
                assert np.array_equal(g.numpy(), layout.concat_bwd(ug, list(shapes), j, dim) + (init if acc else 0))
    t = rng.normal(0, 1, (4, 12, 3)).astype(np.float32)
    sections = [5, 5, 2]
    want = layout.split_fwd(t, sections, 1)
    outs = [ctx.empty(w.shape) for w in want]
    ptrs = (C.c_void_p * 3)(*[a.ptr.value if hasattr(a.ptr, "value") else a.ptr for a in outs])
    sec = (C.c_int64 * 3)(*sections)
    ctx._check(L.mtl_split_fwd(h, ptrs, ctx.array(t).ptr, 3, 3, _shape(t.shape), sec, 1))
    for o, w in zip(outs, want):
        assert np.array_equal(o.numpy(), w)
    ugs = [rng.normal(0, 1, w.shape).astype(np.float32) for w in want]
    dev = [ctx.array(u) for u in ugs]
    ptrs = (C.c_void_p * 3)(*[a.ptr.value if hasattr(a.ptr, "value") else a.ptr for a in dev])
    init = rng.normal(0, 1, t.shape).astype(np.float32)
    for acc in (0, 1):
        g = ctx.array(init)
        ctx._check(L.mtl_split_bwd(h, g.ptr, ptrs, 3, 3, _shape(t.shape), sec, 1, acc))
        assert np.array_equal(g.numpy(), layout.split_bwd(ugs, t.shape, sections, 1) + (init if acc else 0))
    bad = (C.c_int64 * 3)(5, 5, 3)
    assert L.mtl_split_fwd(h, ptrs, ctx.array(t).ptr, 3, 3, _shape(t.shape), bad, 1) != 0


@pytest.mark.gpu
def test_transpose_and_slice_as_graph_nodes(ctx):
    """A small graph through TRANSPOSE and SLICE nodes: loss and parameter gradients of the C++ mirror
    against the oracle's executor (Graph.op with the reference's attribute names)."""
    from mantle_b200 import OP, host_api
    from test_models_gpu import make_pair

    def build(ns, g):
        x = g.input((6, 5))
        y = g.input((3, 4))
        h = ns.nn.Linear(g, x, 8)                                  # [6, 8]
        h = g.op(OP.TRANSPOSE, h)                                  # [8, 6]
        h = g.op(OP.SLICE, h, starts=(1, 5), ends=(8, 0), steps=(2, -2), axes=(0, 1))   # rows 1,3,5,7; cols 5,3,1 -> [4, 3]
        h = g.op(OP.TRANSPOSE, h, axes=(1, 0))                     # [3, 4]
        g.out(h)
        g.loss(ns.nn.MSELoss(g, h, y))

    (g, m), (og, om) = make_pair(ctx, build, seed=61)
    rng = np.random.default_rng(62)
    x = rng.normal(0, 1, (6, 5)).astype(np.float32)
    y = rng.normal(0, 1, (3, 4)).astype(np.float32)
    loss, oloss = m.forward(x, y), om.forward(x, y)
    assert abs(loss - oloss) <= 1e-5 * abs(oloss) + 1e-6
    m.zero_grads(); om.zero_grads()
    m.backward(); om.backward()
    for s, os_ in zip(g.params(), og.params()):
        if s.trainable:
            assert np.allclose(m.grad(s), om.grad(os_), rtol=1e-4, atol=1e-6)
    out_sym = host_api.Symbol(g, g.node(4)["output"])   # Linear = DOT + ADD, then TRANSPOSE, SLICE, TRANSPOSE
    got = m.inference(x, y, outputs=[out_sym])[0]
    assert got.shape == (3, 4) and np.allclose(got, om.inference(x, y)[0], rtol=1e-5, atol=1e-6)


def _build_concat_split(ns, g):
    from mantle_b200 import OP
    x = g.input((4, 6))
    y = g.input((4, 3))
    h = ns.nn.Linear(g, x, 6)                                      # trainable path in front of the SPLIT
    a, b = g.split(h, [2, 4], dim=1)                               # [4, 2], [4, 4]
    h = g.concat(g.op(OP.TANH, b), g.op(OP.RELU, a), a, dim=1)     # [4, 8]: `a` is read twice
    top, rest = g.split(h, [1, 3], dim=0)                          # [1, 8], [3, 8]
    h = g.concat(rest, top, dim=0)                                 # rows rotated
    out = ns.nn.Linear(g, h, 3)
    g.out(out)
    g.loss(ns.nn.MSELoss(g, out, y))
    g.test_out = out


def test_concat_split_nodes_in_the_oracle_executor():
    """Graph.concat / Graph.split (graph.mojo:180-210) in the CPU executor against plain numpy."""
    og = oracle.Graph()
    _build_concat_split(oracle, og)
    om = oracle.Model(og)
    rng = np.random.default_rng(71)
    x = rng.normal(0, 1, (4, 6)).astype(np.float32)
    y = rng.normal(0, 1, (4, 3)).astype(np.float32)
    w1, b1, w2, b2 = [om.tensor(s).astype(np.float64) for s in og.params() if s.trainable]
    h = x @ w1 + b1
    a, b = h[:, :2], h[:, 2:]
    h = np.concatenate([np.tanh(b), np.maximum(a, 0), a], 1)
    h = np.concatenate([h[1:], h[:1]], 0)
    want = np.mean((y - (h @ w2 + b2)) ** 2)
    assert abs(om.forward(x, y) - want) <= 1e-5 * abs(want)
    # gradient of the first weight by central differences through the whole chain
    om.zero_grads(); om.backward()
    s_w1 = [s for s in og.params() if s.trainable][0]
    g_w1 = om.grad(s_w1)
    base = om.tensor(s_w1)
    for (i, j) in ((0, 0), (3, 4), (5, 1)):
        d = np.zeros_like(base); d[i, j] = 1e-2
        om.set_tensor(s_w1, base + d); lp = om.forward(x, y)
        om.set_tensor(s_w1, base - d); lm = om.forward(x, y)
        om.set_tensor(s_w1, base)
        assert abs((lp - lm) / 2e-2 - g_w1[i, j]) <= 2e-2 * abs(g_w1[i, j]) + 2e-3


@pytest.mark.gpu
def test_concat_and_split_as_graph_nodes(ctx):
    """CONCAT (several operands, one read twice) and SPLIT (several results) as nodes of the C++ mirror: loss,
    every parameter gradient and the graph output against the oracle's executor, in both accumulation modes."""
    from test_models_gpu import make_pair
    for strict in (False, True):
        (g, m), (og, om) = make_pair(ctx, _build_concat_split, seed=72)
        m.set_overwrite_first(not strict)
        rng = np.random.default_rng(73)
        x = rng.normal(0, 1, (4, 6)).astype(np.float32)
        y = rng.normal(0, 1, (4, 3)).astype(np.float32)
        loss, oloss = m.forward(x, y), om.forward(x, y)
        assert abs(loss - oloss) <= 1e-5 * abs(oloss) + 1e-6
        m.zero_grads(); om.zero_grads()
        m.backward(); om.backward()
        for s, os_ in zip(g.params(), og.params()):
            if s.trainable:
                assert np.allclose(m.grad(s), om.grad(os_), rtol=1e-4, atol=1e-6), strict
        assert np.allclose(m.inference(x, y, outputs=[g.test_out])[0], om.inference(x, y)[0], rtol=1e-5, atol=1e-6)
    assert ctx.device_status() == 0
