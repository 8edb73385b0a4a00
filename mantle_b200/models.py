"""Graph builders of the networks this backend is measured and tested on, written against the
layer interface of mantle/nn (nn.Linear, nn.Conv2d, nn.MaxPool2d, nn.ReLU, nn.MSELoss,
nn.CrossEntropyLoss) and Graph.input / Graph.op / Graph.out / Graph.loss of
mantle/autograd/graph.mojo.

Every builder takes the namespace `ns` that provides `OP`, `nn` and `Graph` -- `GpuNs` below for the
host mirror of this package; a test passes its CPU checker's namespace to build the identical graph
there -- so that one definition serves both sides of a parity comparison.
"""
from __future__ import annotations

import numpy as np

from . import host_api
from ._lib import OP as _OP


class GpuNs:
    """The host mirror's graph-building namespace (libmantle_host.so behind host_api)."""
    OP = _OP
    nn = host_api.nn
    Graph = host_api.Graph


def build_regression(ns, g, batch=32, features=13):
    """Linear(13 -> 1) trained on MSE: examples/housing.mojo:38-49."""
    x = g.input((batch, features))
    y = g.input((batch, 1))
    out = ns.nn.Linear(g, x, 1)
    g.out(out)
    g.loss(ns.nn.MSELoss(g, out, y))


def build_sin(ns, g, batch=32, hidden=32):
    """Linear(1 -> 32), ReLU, Linear(32 -> 32), ReLU, Linear(32 -> 1) on MSE: examples/sin_estimate.mojo:21-38."""
    x = g.input((batch, 1))
    y = g.input((batch, 1))
    h = ns.nn.ReLU(g, ns.nn.Linear(g, x, hidden))
    h = ns.nn.ReLU(g, ns.nn.Linear(g, h, hidden))
    out = ns.nn.Linear(g, h, 1)
    g.out(out)
    g.loss(ns.nn.MSELoss(g, out, y))


def build_cnn(ns, g, B=4, c1=16, c2=32):
    """Conv(1 -> c1, 5x5, pad 2), ReLU, MaxPool 2x2, Conv(c1 -> c2, 5x5, pad 2), ReLU, MaxPool 2x2,
    Linear(c2*49 -> 10), softmax cross-entropy on 28x28 images: examples/mnist.mojo:33-56.
    c1, c2 = 16, 32 is the example's network; 64, 128 the widened one the throughput is quoted on."""
    x = g.input((B, 1, 28, 28))
    y = g.input((B, 10))
    h = ns.nn.MaxPool2d(g, ns.nn.ReLU(g, ns.nn.Conv2d(g, x, c1, (5, 5), padding=(2, 2))), (2, 2))
    h = ns.nn.MaxPool2d(g, ns.nn.ReLU(g, ns.nn.Conv2d(g, h, c2, (5, 5), padding=(2, 2))), (2, 2))
    h = g.op(ns.OP.RESHAPE, h, shape=(B, c2 * 7 * 7))
    out = ns.nn.Linear(g, h, 10)
    g.out(out)
    g.loss(ns.nn.CrossEntropyLoss(g, out, y))


def fan_in_of(shape, bias_fan_in):
    """fan_in the reference's layers initialise with: C*R*S for a convolution kernel
    (nn/layers/conv.mojo:47-59), rows for a Linear weight (nn/layers/linear.mojo:34-43); a bias takes
    the fan_in of its layer, which the caller passes."""
    if len(shape) == 4:
        return int(np.prod(shape[1:]))
    if len(shape) == 2:
        return int(shape[0])
    return int(bias_fan_in)


def cnn_weights(shapes, seed=43):
    """Seeded U(+-1/sqrt(fan_in)) values for the six trainable tensors of build_cnn, in
    get_trainable_parameters order (W1, b1, W2, b2, W3, b3)."""
    rng = np.random.default_rng(seed)
    out, last = [], 1
    for s in shapes:
        fan = fan_in_of(s, last)
        last = fan
        out.append(rng.uniform(-1, 1, s).astype(np.float32) / np.float32(np.sqrt(fan)))
    return out


def cnn_batch_pool(n, seed=42, one_hot=True):
    """Synthetic stand-in for the MNIST csv of examples/mnist.mojo: pixels ~ U(0,1), labels uniform
    over 0..9, as fp32 labels and (optionally) as the one-hot rows the example builds per batch."""
    rng = np.random.default_rng(seed)
    x = rng.uniform(0.0, 1.0, (n, 1, 28, 28)).astype(np.float32)
    labels = rng.integers(0, 10, n)
    y = np.eye(10, dtype=np.float32)[labels] if one_hot else None
    return x, labels.astype(np.float32), y
