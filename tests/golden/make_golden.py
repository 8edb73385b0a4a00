"""Generates the golden fixtures in this folder with PyTorch CPU.

PyTorch CPU is the oracle the reference's own op and model tests compare against
(tests/python/test_ops_torch.mojo:31-70, test_conv.mojo, test_pool.mojo, test_models_*.mojo with
test_models_torch.py; pinned to torch 2.11 in pixi.lock).  Those tests draw random inputs at run
time, so they hold no stored vectors; this script restates their cases with seeded numpy inputs
and stores inputs and torch's outputs.  The model twins below are written for this repository;
like the reference's twins they use F.linear(x, W.T, b) because Mantle stores Linear weights as
[in, out].

    python tests/golden/make_golden.py        # rewrites tests/golden/*.npz

The fixtures are float32 arrays, about 2.5 MB in total, and are committed.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F

OUT = Path(__file__).resolve().parent
torch.set_num_threads(1)
torch.backends.mkldnn.enabled = False  # plain fp32 reference arithmetic


def t(a, grad=False):
    x = torch.tensor(np.asarray(a, np.float32))
    x.requires_grad_(grad)
    return x


# ---- conv / pool cases: (name, x_shape, w_shape | kernel_size, padding, stride, dilation) ------
# test_conv.mojo:172-234 (forward) and :279-353 (backward); the first two forward cases there use
# constant fills, random inputs are used here for all of them.
CONV_CASES = [
    ("fwd_1x16_p2", (4, 1, 28, 28), (1, 1, 1, 16), (2, 2), (1, 1), (1, 1)),
    ("fwd_2x2_p0", (4, 1, 32, 17), (1, 1, 2, 2), (0, 0), (1, 1), (1, 1)),
    ("fwd_2x2_p31_s23_d23", (4, 3, 32, 17), (2, 3, 2, 2), (3, 1), (2, 3), (2, 3)),
    ("bwd_1x16_p2", (4, 2, 28, 28), (3, 2, 1, 16), (2, 2), (1, 1), (1, 1)),
    ("bwd_4x8_p24_s31_d2", (4, 2, 28, 28), (3, 2, 4, 8), (2, 4), (3, 1), (2, 2)),
    ("bwd_5x6_p32_s2_d32", (4, 2, 28, 28), (3, 2, 5, 6), (3, 2), (2, 2), (3, 2)),
    # the layers of the benchmark CNNs at a tiny batch
    ("cnn_conv1", (2, 1, 28, 28), (16, 1, 5, 5), (2, 2), (1, 1), (1, 1)),
    ("cnn_conv2", (2, 16, 14, 14), (32, 16, 5, 5), (2, 2), (1, 1), (1, 1)),
]
# test_pool.mojo:107-146 (forward), :178-248 (backward)
POOL_CASES = [
    ("k5_p2_s1", (4, 1, 28, 28), (5, 5), (2, 2), (1, 1), (1, 1)),
    ("k2_p0_s1", (4, 1, 32, 17), (2, 2), (0, 0), (1, 1), (1, 1)),
    ("k6_p31_s23_d23", (4, 3, 32, 17), (6, 6), (3, 1), (2, 3), (2, 3)),
    ("k2_s2", (3, 5, 28, 28), (2, 2), (0, 0), (2, 2), (1, 1)),
]


def make_conv_pool(rng):
    out = {}
    for name, xs, ws, pad, st, dil in CONV_CASES:
        x = rng.uniform(0, 1, xs).astype(np.float32)
        w = rng.uniform(-0.5, 0.5, ws).astype(np.float32)
        b = rng.uniform(-0.5, 0.5, ws[0]).astype(np.float32)
        tx, tw, tb = t(x, True), t(w, True), t(b, True)
        y = F.conv2d(tx, tw, tb, stride=st, padding=pad, dilation=dil)
        ug = rng.uniform(0, 1, tuple(y.shape)).astype(np.float32)
        y.backward(t(ug))
        for k, v in dict(x=x, w=w, b=b, y=y.detach().numpy(), ug=ug, dx=tx.grad.numpy(), dw=tw.grad.numpy(),
                         db=tb.grad.numpy(), attrs=np.array(list(pad) + list(st) + list(dil), np.int64)).items():
            out["conv_%s__%s" % (name, k)] = v
    for name, xs, ks, pad, st, dil in POOL_CASES:
        x = rng.uniform(0, 1, xs).astype(np.float32)
        tx = t(x, True)
        y, idx = F.max_pool2d(tx, ks, stride=st, padding=pad, dilation=dil, return_indices=True)
        ug = rng.uniform(0, 1, tuple(y.shape)).astype(np.float32)
        y.backward(t(ug))
        for k, v in dict(x=x, y=y.detach().numpy(), idx=idx.numpy().astype(np.int32), ug=ug, dx=tx.grad.numpy(),
                         attrs=np.array(list(ks) + list(pad) + list(st) + list(dil), np.int64)).items():
            out["pool_%s__%s" % (name, k)] = v
    np.savez_compressed(OUT / "conv_pool.npz", **out)


def make_ops(rng):
    """DOT shapes of test_ops_torch.mojo:254-331 (reduced where large), broadcast elementwise
    (37,63,107)-style cases shrunk, axis reductions."""
    out = {}
    for i, (m, k, n) in enumerate([(107, 203, 139), (107, 186, 107), (64, 128, 256), (32, 13, 1)]):
        a = rng.uniform(0, 1, (m, k)).astype(np.float32)
        b = rng.uniform(0, 1, (k, n)).astype(np.float32)
        ta, tb = t(a, True), t(b, True)
        c = ta @ tb
        ug = rng.uniform(0, 1, (m, n)).astype(np.float32)
        c.backward(t(ug))
        out.update({"dot%d__a" % i: a, "dot%d__b" % i: b, "dot%d__c" % i: c.detach().numpy(), "dot%d__ug" % i: ug,
                    "dot%d__da" % i: ta.grad.numpy(), "dot%d__db" % i: tb.grad.numpy()})
    ops = {"add": torch.add, "sub": torch.sub, "mul": torch.mul, "div": torch.div}
    shapes = [((7, 13, 17), (7, 13, 17)), ((7, 13, 17), (7, 13, 1)), ((32, 10), (10,)), ((32, 10), (32, 1)),
              ((5, 1, 6), (4, 1)), ((6, 5), (1,))]
    for name, fn in ops.items():
        for j, (sa, sb) in enumerate(shapes):
            a = rng.uniform(0.5, 1.5, sa).astype(np.float32)
            b = rng.uniform(0.5, 1.5, sb).astype(np.float32)
            ta, tb = t(a, True), t(b, True)
            c = fn(ta, tb)
            ug = rng.uniform(0, 1, tuple(c.shape)).astype(np.float32)
            c.backward(t(ug))
            key = "bin_%s%d" % (name, j)
            out.update({key + "__a": a, key + "__b": b, key + "__c": c.detach().numpy(), key + "__ug": ug,
                        key + "__da": ta.grad.numpy(), key + "__db": tb.grad.numpy()})
    un = {"exp": torch.exp, "log": torch.log, "sigmoid": torch.sigmoid, "relu": torch.relu, "tanh": torch.tanh,
          "pow2": lambda x: x ** 2, "pow3": lambda x: x ** 3,
          "leakyrelu": lambda x: F.leaky_relu(x, 0.1), "clip": lambda x: torch.clamp(x, -0.3, 0.4)}
    for name, fn in un.items():
        x = rng.uniform(0.2, 2.0, (9, 11)).astype(np.float32) if name == "log" else rng.normal(0, 1, (9, 11)).astype(np.float32)
        tx = t(x, True)
        y = fn(tx)
        ug = rng.uniform(0, 1, (9, 11)).astype(np.float32)
        y.backward(t(ug))
        out.update({"un_%s__x" % name: x, "un_%s__y" % name: y.detach().numpy(), "un_%s__ug" % name: ug,
                    "un_%s__dx" % name: tx.grad.numpy()})
    x = rng.normal(0, 1, (8, 7, 10)).astype(np.float32)
    out["red__x"] = x
    for name, fn in {"sum": torch.sum, "mean": torch.mean}.items():
        for axis in (None, 0, 1, 2):
            tx = t(x, True)
            y = fn(tx) if axis is None else fn(tx, dim=axis, keepdim=True)
            y = y.reshape(1) if axis is None else y
            ug = rng.uniform(0, 1, tuple(y.shape)).astype(np.float32)
            y.backward(t(ug))
            key = "red_%s_%s" % (name, "all" if axis is None else axis)
            out.update({key + "__y": y.detach().numpy(), key + "__ug": ug, key + "__dx": tx.grad.numpy()})
    for axis in (None, 0, 1, 2):
        tx = t(x, True)
        y = tx.max().reshape(1) if axis is None else tx.max(dim=axis, keepdim=True).values
        ug = rng.uniform(0, 1, tuple(y.shape)).astype(np.float32)
        y.backward(t(ug))  # no ties in continuous random data
        key = "red_max_%s" % ("all" if axis is None else axis)
        out.update({key + "__y": y.detach().numpy(), key + "__ug": ug, key + "__dx": tx.grad.numpy()})
    np.savez_compressed(OUT / "ops.npz", **out)


def adam(params, lr):
    return torch.optim.Adam(params, lr=lr, betas=(0.9, 0.999), eps=1e-8)


def make_models(rng):
    """100-step loss trajectories on one fixed batch, as test_models_{regression,sin_estimate,mnist}
    do (Adam, identical literal weights on both sides)."""
    out = {}
    # regression: Linear(13 -> 1), MSE, batch 32 (the shape of examples/housing.mojo), lr 0.05
    x = rng.normal(0, 1, (32, 13)).astype(np.float32)
    w_true = rng.normal(0, 1, 13).astype(np.float32)
    y = (x @ w_true + 20.0 + rng.normal(0, 0.5, 32)).astype(np.float32).reshape(32, 1)
    W = rng.uniform(-0.27, 0.27, (13, 1)).astype(np.float32)
    b = rng.uniform(-0.27, 0.27, 1).astype(np.float32)
    out.update(reg__x=x, reg__y=y, reg__W=W, reg__b=b)
    ps = [t(W, True), t(b, True)]
    opt = adam(ps, 0.05)
    losses = []
    for _ in range(100):
        loss = F.mse_loss(F.linear(t(x), ps[0].T, ps[1]), t(y))
        opt.zero_grad(); loss.backward(); opt.step()
        losses.append(loss.item())
    out["reg__losses"] = np.array(losses, np.float32)
    out["reg__W_final"] = ps[0].detach().numpy()

    # sine MLP 1 -> 32 -> 32 -> 1, MSE, batch 32, lr 0.01
    x = rng.uniform(-np.pi, np.pi, (32, 1)).astype(np.float32)
    y = np.sin(x).astype(np.float32)
    dims = [(1, 32), (32, 32), (32, 1)]
    ws = []
    for fi, fo in dims:
        bnd = 1.0 / np.sqrt(fi)
        ws += [rng.uniform(-bnd, bnd, (fi, fo)).astype(np.float32), rng.uniform(-bnd, bnd, fo).astype(np.float32)]
    out.update(sin__x=x, sin__y=y, **{"sin__p%d" % i: w for i, w in enumerate(ws)})
    ps = [t(w, True) for w in ws]
    opt = adam(ps, 0.01)
    losses = []
    for _ in range(100):
        h = torch.relu(F.linear(t(x), ps[0].T, ps[1]))
        h = torch.relu(F.linear(h, ps[2].T, ps[3]))
        loss = F.mse_loss(F.linear(h, ps[4].T, ps[5]), t(y))
        opt.zero_grad(); loss.backward(); opt.step()
        losses.append(loss.item())
    out["sin__losses"] = np.array(losses, np.float32)

    # CNN of examples/mnist.mojo, cross entropy written as -sum(t * log_softmax) / N, lr 1e-3.
    # test_models_mnist.mojo:229-295 sets every weight to 0.02: the gradient reaching the layers
    # below the classifier is then pure rounding noise (the class gradients of a sample sum to
    # zero), which Adam's normalisation amplifies, so seeded U(+-1/sqrt(fan_in)) weights are used.
    # Batch 16 stays within 1e-3 relative of this twin over 100 steps under fp32 re-orderings;
    # batch 4 (the reference's size) overfits to ~2e-3 within 100 steps and is compared for 30.
    for tag, B in (("cnn", 16), ("cnn4", 4)):
        x = rng.uniform(0, 1, (B, 1, 28, 28)).astype(np.float32)
        y = np.eye(10, dtype=np.float32)[rng.integers(0, 10, B)]
        shapes = [(16, 1, 5, 5), (16,), (32, 16, 5, 5), (32,), (1568, 10), (10,)]
        fans = [25, 25, 400, 400, 1568, 1568]
        ws = [rng.uniform(-1 / np.sqrt(f), 1 / np.sqrt(f), s).astype(np.float32) for s, f in zip(shapes, fans)]
        out.update({tag + "__x": x, tag + "__y": y}, **{"%s__p%d" % (tag, i): w for i, w in enumerate(ws)})
        ps = [t(w, True) for w in ws]
        opt = adam(ps, 1e-3)
        losses = []
        for _ in range(100):
            h = F.max_pool2d(torch.relu(F.conv2d(t(x), ps[0], ps[1], padding=2)), 2)
            h = F.max_pool2d(torch.relu(F.conv2d(h, ps[2], ps[3], padding=2)), 2)
            o = F.linear(h.reshape(B, -1), ps[4].T, ps[5])
            loss = -torch.sum(t(y) * F.log_softmax(o, dim=1)) / B
            opt.zero_grad(); loss.backward(); opt.step()
            losses.append(loss.item())
        out[tag + "__losses"] = np.array(losses, np.float32)
    np.savez_compressed(OUT / "models.npz", **out)


if __name__ == "__main__":
    make_conv_pool(np.random.default_rng(42))
    make_ops(np.random.default_rng(43))
    make_models(np.random.default_rng(44))
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size, "bytes")
