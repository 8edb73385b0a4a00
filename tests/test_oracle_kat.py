"""Pins the CPU oracle: known-answer values restated from the reference's own tests
(tests/mojo/test_ops.mojo, test_backward.mojo, test_mlops.mojo, test_activations.mojo,
test_loss.mojo, test_tensorutils.mojo, tests/python/test_conv.mojo shape cases) and the PyTorch-CPU
fixtures of tests/golden (the oracle the reference's tests/python files use).  CPU only."""
import math

import numpy as np
import pytest

import oracle
from mantle_b200.models import build_cnn, build_regression, build_sin
from oracle import OP, nn
from helpers import assert_close, cases, golden


def full(shape, v):
    return np.full(shape, v, np.float32)


# ---- tests/mojo/test_ops.mojo:13-196 -----------------------------------------------------------
def test_elementwise_forward_kat():
    assert_close(oracle.forward_op(OP.ADD, full((2, 3), 1), full((2, 3), 1)), full((2, 3), 2))
    assert_close(oracle.forward_op(OP.SUB, full((2, 3), 2), full((2, 3), 1)), full((2, 3), 1))
    assert_close(oracle.forward_op(OP.MUL, full((2, 3), 2), full((2, 3), 3)), full((2, 3), 6))
    assert_close(oracle.forward_op(OP.DIV, full((2, 3), 6), full((2, 3), 2)), full((2, 3), 3))
    assert_close(oracle.forward_op(OP.EXP, full((2, 3), 2)), full((2, 3), math.exp(2)))
    assert_close(oracle.forward_op(OP.LOG, full((2, 3), 2)), full((2, 3), math.log(2)))
    assert_close(oracle.forward_op(OP.POW, full((2, 3), 2), exponent=2), full((2, 3), 4))


def test_dot_kat():
    # test_ops.mojo:69-80, test_tensorutils.mojo:47-66
    assert_close(oracle.dot(full((2, 3), 1), full((3, 2), 2)), full((2, 2), 6))
    # test_backward.mojo:96-113
    assert_close(oracle.dot_transpose_t2(full((2, 2), 1), full((3, 2), 2)), full((2, 3), 4))
    assert_close(oracle.dot_transpose_t1(full((2, 3), 1), full((2, 2), 1)), full((3, 2), 2))


def test_reduce_forward_kat():
    t = full((2, 3, 4), 1)
    assert_close(oracle.reduce_fwd(OP.SUM, t), full((1,), 24))
    assert_close(oracle.reduce_fwd(OP.SUM, t, 1), full((2, 1, 4), 3))
    t = np.arange(1, 13, dtype=np.float32).reshape(2, 3, 2)
    assert_close(oracle.reduce_fwd(OP.MAX, t), full((1,), 12))
    assert_close(oracle.reduce_fwd(OP.MAX, t, 0).ravel(), [7, 8, 9, 10, 11, 12])
    assert_close(oracle.reduce_fwd(OP.MAX, t, 1).ravel(), [5, 6, 11, 12])
    assert_close(oracle.reduce_fwd(OP.MAX, t, 2).ravel(), [2, 4, 6, 8, 10, 12])
    t = full((2, 3), 5)
    assert_close(oracle.reduce_fwd(OP.MEAN, t), full((1,), 5))
    assert_close(oracle.reduce_fwd(OP.MEAN, t, 0), full((1, 3), 5))
    assert_close(oracle.reduce_fwd(OP.MEAN, t, 1), full((2, 1), 5))


# ---- tests/mojo/test_backward.mojo:18-358 ------------------------------------------------------
def test_binary_backward_kat():
    ug = full((2, 3), 1)
    for op, a, b, g1, g2 in [(OP.ADD, 1, 2, 1, 1), (OP.SUB, 2, 1, 1, -1), (OP.MUL, 1, 2, 2, 1),
                             (OP.DIV, 1, 2, 0.5, -0.25)]:
        assert_close(oracle.backward_op(0, op, ug, full((2, 3), a), full((2, 3), b)), full((2, 3), g1))
        assert_close(oracle.backward_op(1, op, ug, full((2, 3), a), full((2, 3), b)), full((2, 3), g2))


def test_unary_backward_kat():
    assert_close(oracle.backward_op(0, OP.EXP, full((2, 3), 5), full((2, 3), 2)), full((2, 3), 5 * math.exp(2)))
    assert_close(oracle.backward_op(0, OP.LOG, full((2, 3), 5), full((2, 3), 2)), full((2, 3), 2.5))
    assert_close(oracle.backward_op(0, OP.POW, full((2, 3), 1), full((2, 3), 2), exponent=2), full((2, 3), 4))
    # test_mlops.mojo:53-90 and the sigmoid case above it
    t = np.array([[3, 3, 3], [-3, -3, -3]], np.float32)
    assert_close(oracle.forward_op(OP.RELU, t), np.array([[3, 3, 3], [0, 0, 0]], np.float32))
    assert_close(oracle.backward_op(0, OP.RELU, full((2, 3), 5), t), np.array([[5, 5, 5], [0, 0, 0]], np.float32))
    assert_close(oracle.backward_op(0, OP.SIGMOID, full((2, 3), 5), full((2, 3), 0)), full((2, 3), 1.25))


def test_pow_exponent_backward_kat():
    # test_backward.mojo:142-168: d(x^a)/da summed over the tensor; log(0) counts as 0
    want = np.array([6 * 4 * math.log(2.0)], np.float32)
    assert_close(oracle.backward_op(1, OP.POW, full((2, 3), 1), full((2, 3), 2), exponent=2), want)
    assert_close(oracle.backward_op(1, OP.POW, full((2, 3), 1), full((2, 3), 0), exponent=0), np.zeros(1, np.float32))
    assert_close(oracle.backward_op(0, OP.POW, full((2, 3), 1), full((2, 3), 0), exponent=0), full((2, 3), 0))
    # accumulation into an existing gradient (ops.mojo:463)
    g = np.array([1.5], np.float32)
    oracle.backward_op(1, OP.POW, full((2, 3), 1), full((2, 3), 2), exponent=2, grad=g)
    assert_close(g, want + 1.5)


def test_fma_kat():
    # tests/mojo/test_ops.mojo:256-270
    assert_close(oracle.forward_op(OP.FMA, full((2, 3), 1), full((2, 3), 2), full((2, 3), 3)), full((2, 3), 5))
    # tests/python/test_ops_torch.mojo:881-905 (torch: t1 * t2 + t3, upper gradient t1) at its shape
    rng = np.random.default_rng(11)
    t1, t2, t3 = (rng.uniform(0, 1, (87, 73, 84)).astype(np.float32) for _ in range(3))
    assert_close(oracle.forward_op(OP.FMA, t1, t2, t3), t1 * t2 + t3, 1e-5, 1e-6)
    for tid, want in enumerate((t1 * t2, t1 * t1, t1)):
        assert_close(oracle.backward_op(tid, OP.FMA, t1, t1, t2, t3), want, 1e-6, 1e-7, "FMA grad %d" % tid)


def test_reduce_backward_kat():
    assert_close(oracle.backward_op(0, OP.SUM, full((1,), 9), full((2, 3), 1)), full((2, 3), 9))
    ug = np.array([[0, 1, 2]], np.float32)
    assert_close(oracle.backward_op(0, OP.SUM, ug, full((2, 3), 1), axis=0).ravel(), [0, 1, 2, 0, 1, 2])
    ug = np.array([[0], [1]], np.float32)
    assert_close(oracle.backward_op(0, OP.SUM, ug, full((2, 3), 1), axis=1).ravel(), [0, 0, 0, 1, 1, 1])
    assert_close(oracle.backward_op(0, OP.MEAN, full((1,), 9), full((2, 3), 1)), full((2, 3), 1.5))
    assert_close(oracle.backward_op(0, OP.MEAN, full((1, 3), 3), full((2, 3), 1), axis=0), full((2, 3), 1.5))
    assert_close(oracle.backward_op(0, OP.MEAN, full((2, 1), 3), full((2, 3), 1), axis=1), full((2, 3), 1.0))


def test_max_backward_ties_kat():
    # test_backward.mojo:222-309: the gradient is split 1/n between n tied maxima
    t = full((2, 3), 1)
    t[0, 0] = t[0, 1] = 2
    want = np.zeros((2, 3), np.float32)
    want[0, 0] = want[0, 1] = 4.5
    assert_close(oracle.backward_op(0, OP.MAX, full((1,), 9), t), want)
    base = np.arange(1, 13, dtype=np.float32).reshape(2, 3, 2)
    t = base.copy(); t.ravel()[0] = 7
    want = np.zeros(12, np.float32); want[[0, 6]] = 1; want[7:12] = 2
    assert_close(oracle.backward_op(0, OP.MAX, full((1, 3, 2), 2), t, axis=0).ravel(), want)
    t = base.copy(); t.ravel()[0] = 5
    want = np.zeros(12, np.float32); want[[0, 4]] = 1; want[[5, 10, 11]] = 2
    assert_close(oracle.backward_op(0, OP.MAX, full((2, 1, 2), 2), t, axis=1).ravel(), want)
    t = base.copy(); t.ravel()[0] = 2
    want = np.zeros(12, np.float32); want[[0, 1]] = 1; want[[3, 5, 7, 9, 11]] = 2
    assert_close(oracle.backward_op(0, OP.MAX, full((2, 3, 1), 2), t, axis=2).ravel(), want)


def test_unbroadcast_kat():
    # accumulate_grad un-broadcasting, test_tensorutils.mojo:397-417: [2,3,4] of 3.0 into [2,1,1] -> 36
    a = full((2, 3, 4), 3)
    g = oracle.binary_bwd(OP.ADD, 1, a, np.zeros((2, 3, 4), np.float32), np.zeros((2, 1, 1), np.float32))
    assert_close(g, full((2, 1, 1), 36))


# ---- tests/mojo/test_activations.mojo:105-140, test_loss.mojo ----------------------------------
@pytest.mark.parametrize("axis,soft,logsoft", [(0, 0.5, -0.69314718), (1, 1 / 3, -1.09861231), (2, 0.5, -0.69314718)])
def test_softmax_kat(axis, soft, logsoft):
    for builder, want, nodes in [(nn.Softmax, soft, 5), (nn.LogSoftmax, logsoft, 6)]:
        g = oracle.Graph()
        x = g.input((2, 3, 2))
        out = builder(g, x, axis)
        g.out(out)
        assert g.counts()["nodes"] == nodes
        res = oracle.Model(g).inference(full((2, 3, 2), 4))[0]
        assert_close(res, full((2, 3, 2), want))


def _ce_graph():
    g = oracle.Graph()
    yp, yt = g.input((2, 3)), g.input((2, 3))
    g.out(nn.CrossEntropyLoss(g, yp, yt))
    return g


def test_cross_entropy_kat():
    g = _ce_graph()
    assert g.counts()["nodes"] == 9  # test_loss.mojo:102
    yp = np.array([[0.1, 0.2, 0.7], [0.7, 0.2, 0.1]], np.float32)
    loss = oracle.Model(g).inference(yp, np.array([[0, 0, 1], [1, 0, 0]], np.float32))[0]
    assert loss.shape == (1,)
    assert_close(loss, [0.76794958])  # test_loss.mojo:127
    loss = oracle.Model(_ce_graph()).inference(yp, np.array([[0, 1, 0], [0, 0, 1]], np.float32))[0]
    assert_close(loss, [1.31794953])  # test_loss.mojo:171


def test_mse_kat():
    g = oracle.Graph()
    yp, yt = g.input((64, 10)), g.input((64, 10))
    g.out(nn.MSELoss(g, yp, yt))
    assert g.counts()["nodes"] == 3  # test_loss.mojo:26
    assert_close(oracle.Model(g).inference(full((64, 10), 1), full((64, 10), 1))[0], [0.0])


def test_conv_result_shape_kat():
    # tests/python/test_conv.mojo:17-64
    assert oracle.conv_out_shape((1, 4, 28, 28), 1, 16, (2, 2), (1, 1), (1, 1)) == (32, 17)
    assert oracle.conv_out_shape((1, 4, 32, 17), 2, 2, (0, 0), (1, 1), (1, 1)) == (31, 16)
    assert oracle.conv_out_shape((1, 4, 32, 17), 2, 2, (3, 1), (1, 1), (2, 2)) == (36, 17)
    assert oracle.conv_out_shape((1, 4, 32, 17), 3, 2, (3, 2), (2, 1), (2, 3)) == (17, 18)


# ---- PyTorch-CPU fixtures ----------------------------------------------------------------------
def test_conv_against_torch():
    z = golden("conv_pool")
    for name in cases(z, "conv_"):
        f = lambda k: z["conv_%s__%s" % (name, k)]
        a = f("attrs")
        kw = dict(padding=tuple(a[0:2]), stride=tuple(a[2:4]), dilation=tuple(a[4:6]))
        assert_close(oracle.conv2d_fwd(f("x"), f("w"), f("b"), **kw), f("y"), 1e-4, 1e-5, name + " fwd")
        assert_close(oracle.conv2d_bwd(0, f("ug"), f("x"), f("w"), **kw), f("dx"), 1e-4, 1e-4, name + " dx")
        assert_close(oracle.conv2d_bwd(1, f("ug"), f("x"), f("w"), **kw), f("dw"), 1e-4, 1e-3, name + " dw")
        assert_close(oracle.conv2d_bwd(2, f("ug"), f("x"), f("w"), **kw), f("db"), 1e-4, 1e-3, name + " db")


def test_pool_against_torch():
    z = golden("conv_pool")
    for name in cases(z, "pool_"):
        f = lambda k: z["pool_%s__%s" % (name, k)]
        a = f("attrs")
        kw = dict(kernel_size=tuple(a[0:2]), padding=tuple(a[2:4]), stride=tuple(a[4:6]), dilation=tuple(a[6:8]))
        y, idx = oracle.maxpool2d_fwd(f("x"), return_indices=True, **kw)
        assert np.array_equal(y, f("y")), name          # selection of an input value: exact
        assert np.array_equal(idx, f("idx")), name      # plane-local argmax, as torch reports it
        assert_close(oracle.maxpool2d_bwd(f("ug"), f("x"), **kw), f("dx"), 1e-6, 1e-6, name + " dx")


def test_ops_against_torch():
    z = golden("ops")
    for name in cases(z, "dot"):
        f = lambda k: z["dot%s__%s" % (name, k)]
        assert_close(oracle.dot(f("a"), f("b")), f("c"), 1e-5, 1e-5, "dot" + name)
        assert_close(oracle.dot_transpose_t2(f("ug"), f("b")), f("da"), 1e-5, 1e-5, "dot da" + name)
        assert_close(oracle.dot_transpose_t1(f("a"), f("ug")), f("db"), 1e-5, 1e-5, "dot db" + name)
    opid = {"add": OP.ADD, "sub": OP.SUB, "mul": OP.MUL, "div": OP.DIV}
    for name in cases(z, "bin_"):
        f = lambda k: z["bin_%s__%s" % (name, k)]
        op = opid[name[:3]]
        assert_close(oracle.binary_fwd(op, f("a"), f("b")), f("c"), what=name)
        assert_close(oracle.binary_bwd(op, 0, f("ug"), f("a"), f("b")), f("da"), 1e-5, 1e-4, name + " da")
        assert_close(oracle.binary_bwd(op, 1, f("ug"), f("a"), f("b")), f("db"), 1e-5, 1e-4, name + " db")
    un = {"exp": (OP.EXP, {}), "log": (OP.LOG, {}), "sigmoid": (OP.SIGMOID, {}), "relu": (OP.RELU, {}),
          "tanh": (OP.TANH, {}), "pow2": (OP.POW, {"exponent": 2}), "pow3": (OP.POW, {"exponent": 3}),
          "leakyrelu": (OP.LEAKYRELU, {"negative_slope": 0.1}), "clip": (OP.CLIP, {"min": -0.3, "max": 0.4})}
    for name, (op, kw) in un.items():
        f = lambda k: z["un_%s__%s" % (name, k)]
        assert_close(oracle.forward_op(op, f("x"), **kw), f("y"), 1e-5, 1e-6, name)
        assert_close(oracle.backward_op(0, op, f("ug"), f("x"), **kw), f("dx"), 1e-5, 1e-5, name + " dx")
    x = z["red__x"]
    for rname, op in (("sum", OP.SUM), ("mean", OP.MEAN), ("max", OP.MAX)):
        for axis in (None, 0, 1, 2):
            key = "red_%s_%s" % (rname, "all" if axis is None else axis)
            assert_close(oracle.reduce_fwd(op, x, axis), z[key + "__y"], 1e-5, 1e-5, key)
            assert_close(oracle.reduce_bwd(op, z[key + "__ug"], x, axis), z[key + "__dx"], 1e-5, 1e-6, key + " dx")


def _train(model, opt, inputs, steps):
    losses = []
    for _ in range(steps):
        losses.append(model.forward(*inputs))
        opt.zero_grad()
        model.backward()
        opt.step()
    return np.array(losses, np.float32)


TRAJ = [("reg", build_regression, 0.05, 1e-4, 100), ("sin", build_sin, 0.01, 1e-4, 100),
        ("cnn", lambda ns, g: build_cnn(ns, g, 16), 1e-3, 1e-3, 100), ("cnn4", build_cnn, 1e-3, 1e-3, 30)]


def load_weights(z, name, n):
    return [z["reg__W"], z["reg__b"]] if name == "reg" else [z["%s__p%d" % (name, i)] for i in range(n)]


@pytest.mark.parametrize("name,builder,lr,rtol,steps", TRAJ)
def test_model_trajectories_against_torch(name, builder, lr, rtol, steps):
    """Adam steps on a fixed batch; per-step loss vs the PyTorch twin.  tests/python/test_models_*.mojo
    use rtol 1e-4 (MLPs) and 1e-5 (CNN with constant weights); the CNN here is held to the 1e-3 that
    separates two fp32 implementations with different summation orders after 100 Adam steps."""
    z = golden("models")
    g = oracle.Graph()
    builder(oracle, g)
    m = oracle.Model(g)
    trainable = [s for s in g.params() if s.trainable]
    for s, w in zip(trainable, load_weights(z, name, len(trainable))):
        m.set_tensor(s, w)
    losses = _train(m, oracle.Adam(m, lr=lr), (z[name + "__x"], z[name + "__y"]), steps)
    assert_close(losses, z[name + "__losses"][:steps], rtol, 1e-6, name + " losses")


def test_one_hot_restatement():
    """examples/mnist.mojo:92-97 and the label pattern of test_models_mnist.mojo (label i for sample i)."""
    assert np.array_equal(oracle.one_hot(np.arange(4, dtype=np.float32), 10), np.eye(10, dtype=np.float32)[:4])
    got = oracle.one_hot(np.array([9.0, 0.0, 3.99], np.float32), 10)
    assert got.shape == (3, 10) and got.sum() == 3 and got[0, 9] == 1 and got[1, 0] == 1 and got[2, 3] == 1
