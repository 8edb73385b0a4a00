"""Restatement of Mantle's graph IR, executor and optimizer on the CPU oracle
(TEST INFRASTRUCTURE ONLY).

    Graph / Symbol      mantle/autograd/graph.mojo:40-217, symbol.mojo:61
    nn.*                mantle/nn/layers/{linear,conv,pool}.mojo, activations.mojo, loss.mojo
    Model               mantle/nn/model.mojo:61-395
    Adam                mantle/nn/optim.mojo:27-149

The method names match mantle_b200.host_api so that a test can build the same graph on both."""
from __future__ import annotations

import math
from typing import Optional, Sequence

import numpy as np

from . import layout, ops
from .ops import OP


class Symbol:
    def __init__(self, sid: int, shape: Sequence[int], trainable: bool):
        self.id, self.shape, self.trainable = sid, tuple(int(s) for s in shape), bool(trainable)

    def __repr__(self):
        return "Symbol(%d, %s, trainable=%s)" % (self.id, self.shape, self.trainable)


class Node:
    def __init__(self, op, inputs, outputs, attrs):
        self.op, self.inputs, self.outputs, self.attrs = op, list(inputs), list(outputs), dict(attrs)


def _conv_out(in_shape, R, S, padding, stride, dilation):
    return ops.conv_out_shape(in_shape, R, S, padding, stride, dilation)


def static_result_shape(op, operands, attrs):
    """ops.mojo:104-218"""
    s = [o.shape for o in operands]
    if op in (OP.ADD, OP.SUB, OP.MUL, OP.DIV):
        return ops.broadcast_shapes(s[0], s[1])
    if op in (OP.POW, OP.EXP, OP.LOG, OP.SIGMOID, OP.RELU, OP.LEAKYRELU, OP.TANH, OP.CLIP, OP.FMA):
        return s[0]
    if op == OP.DOT:
        return (s[0][0], s[1][1])
    if op in (OP.SUM, OP.MEAN, OP.MAX):
        axis = attrs.get("axis")
        if axis is None:
            return (1,)
        return tuple(1 if i == axis else d for i, d in enumerate(s[0]))
    if op == OP.FLATTEN:
        return (s[0][0], int(np.prod(s[0])) // s[0][0])
    if op == OP.RESHAPE:
        return tuple(attrs["shape"])
    if op == OP.SQUEEZE:
        dims = attrs.get("dims")
        return tuple(d for i, d in enumerate(s[0]) if not ((dims is None and d == 1) or (dims and i in dims and d == 1)))
    if op == OP.UNSQUEEZE:
        dims = list(attrs.get("dims") or [])
        new_rank = len(s[0]) + len(dims)
        out, j = [], 0
        for i in range(new_rank):
            if i in dims or i - new_rank in dims:
                out.append(1)
            else:
                out.append(s[0][j])
                j += 1
        return tuple(out)
    if op == OP.CONV2D:
        oh, ow = _conv_out(s[0], s[1][2], s[1][3], attrs.get("padding", (0, 0)), attrs.get("stride", (1, 1)),
                           attrs.get("dilation", (1, 1)))
        return (s[0][0], s[1][0], oh, ow)
    if op == OP.MAXPOOL2D:
        k = attrs["kernel_size"]
        oh, ow = _conv_out(s[0], k[0], k[1], attrs.get("padding", (0, 0)), attrs.get("stride", k),
                           attrs.get("dilation", (1, 1)))
        return (s[0][0], s[0][1], oh, ow)
    if op == OP.TRANSPOSE:
        axes = attrs.get("axes") or tuple(range(len(s[0]) - 1, -1, -1))
        return tuple(s[0][a] for a in axes)
    if op == OP.SLICE:
        from . import layout
        return tuple(layout.slice_plan(s[0], attrs["starts"], attrs["ends"], attrs.get("steps"), attrs.get("axes"))[2])
    raise NotImplementedError("operator %d" % op)


class Graph:
    def __init__(self):
        self.inputs, self.param_syms, self.param_inits, self.nodes, self.outputs = [], [], [], [], []
        self.loss_out: Optional[Symbol] = None
        self.symbol_count = 0

    def _create(self, shape, init, trainable, is_input):
        s = Symbol(self.symbol_count, shape, trainable)
        self.symbol_count += 1
        if is_input:
            self.inputs.append(s)
        else:
            self.param_syms.append(s)
            self.param_inits.append(init)
        return s

    def input(self, shape, trainable=False):
        return self._create(shape, None, trainable, True)

    def param(self, shape, init=None, trainable=True):
        return self._create(shape, init, trainable, False)

    def scalar(self, value):
        return self._create((1,), np.array([value], np.float32), False, False)

    def out(self, s):
        self.outputs.append(s)

    def loss(self, s):
        self.loss_out = s

    def op(self, op, *operands, **attrs):
        attrs = {k: v for k, v in attrs.items() if v is not None}
        if len(operands) == 2 and isinstance(operands[1], (int, float)):
            operands = (operands[0], self.scalar(np.float32(operands[1])))
        elif len(operands) == 2 and isinstance(operands[0], (int, float)):
            operands = (self.scalar(np.float32(operands[0])), operands[1])
        shape = static_result_shape(op, operands, attrs)
        res = Symbol(self.symbol_count, shape, any(o.trainable for o in operands))
        self.symbol_count += 1
        self.nodes.append(Node(op, operands, [res], attrs))
        return res

    def concat(self, *operands, dim=0):
        """graph.mojo:180-193."""
        shape = list(operands[0].shape)
        shape[dim] = sum(o.shape[dim] for o in operands)
        res = Symbol(self.symbol_count, tuple(shape), any(o.trainable for o in operands))
        self.symbol_count += 1
        self.nodes.append(Node(OP.CONCAT, operands, [res], {"dim": dim}))
        return res

    def split(self, operand, sections, dim=0):
        """graph.mojo:200-210: one result symbol per section."""
        assert sum(sections) == operand.shape[dim]
        outs = []
        for s in sections:
            shape = tuple(s if a == dim else d for a, d in enumerate(operand.shape))
            outs.append(Symbol(self.symbol_count, shape, operand.trainable))
            self.symbol_count += 1
        self.nodes.append(Node(OP.SPLIT, (operand,), outs, {"sections": list(sections), "dim": dim}))
        return outs

    def counts(self):
        return {"nodes": len(self.nodes), "params": len(self.param_syms), "inputs": len(self.inputs),
                "symbols": self.symbol_count}

    def params(self):
        return list(self.param_syms)


class nn:
    @staticmethod
    def _bound(fan_in):
        return 1.0 / math.sqrt(float(fan_in))

    @staticmethod
    def Linear(g, inputs, n_outputs):
        b = nn._bound(inputs.shape[1])
        w = g.param((inputs.shape[1], n_outputs), ("random_uniform", -b, b))
        bias = g.param((n_outputs,), ("random_uniform", -b, b))
        return g.op(OP.ADD, g.op(OP.DOT, inputs, w), bias)

    @staticmethod
    def Conv2d(g, inputs, out_channels, kernel_size, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
        b = nn._bound(inputs.shape[1] * kernel_size[0] * kernel_size[1])
        w = g.param((out_channels, inputs.shape[1], kernel_size[0], kernel_size[1]), ("random_uniform", -b, b))
        bias = g.param((out_channels,), ("random_uniform", -b, b))
        return g.op(OP.CONV2D, inputs, w, bias, padding=tuple(padding), stride=tuple(stride), dilation=tuple(dilation))

    @staticmethod
    def MaxPool2d(g, inputs, kernel_size, stride=None, padding=(0, 0), dilation=(1, 1)):
        if stride is None:
            stride = kernel_size
        elif isinstance(stride, int):
            stride = (stride, stride)
        return g.op(OP.MAXPOOL2D, inputs, kernel_size=tuple(kernel_size), padding=tuple(padding), stride=tuple(stride),
                    dilation=tuple(dilation))

    @staticmethod
    def ReLU(g, x):
        return g.op(OP.RELU, x)

    @staticmethod
    def Sigmoid(g, x):
        return g.op(OP.SIGMOID, x)

    @staticmethod
    def Tanh(g, x):
        return g.op(OP.TANH, x)

    @staticmethod
    def Softmax(g, x, axis):
        mx = g.op(OP.MAX, x, axis=axis)
        xm = g.op(OP.SUB, x, mx)
        ex = g.op(OP.EXP, xm)
        sm = g.op(OP.SUM, ex, axis=axis)
        return g.op(OP.DIV, ex, sm)

    @staticmethod
    def LogSoftmax(g, x, axis):
        mx = g.op(OP.MAX, x, axis=axis)
        xm = g.op(OP.SUB, x, mx)
        ex = g.op(OP.EXP, xm)
        sm = g.op(OP.SUM, ex, axis=axis)
        lg = g.op(OP.LOG, sm)
        return g.op(OP.SUB, xm, lg)

    @staticmethod
    def MSELoss(g, y_pred, y_true):
        diff = g.op(OP.SUB, y_true, y_pred)
        loss = g.op(OP.POW, diff, 2)
        return g.op(OP.MEAN, loss)

    @staticmethod
    def CrossEntropyLoss(g, y_pred, y_true):
        ls = nn.LogSoftmax(g, y_pred, 1)
        t = g.op(OP.MUL, y_true, ls)
        ret = g.op(OP.SUM, t)
        return g.op(OP.MUL, ret, -1.0 / float(y_pred.shape[0]))


class Model:
    def __init__(self, graph: Graph, seed: int = 42):
        self.g = graph
        self.tensors, self.grads = {}, {}
        rng = np.random.default_rng(seed)
        for s in graph.inputs:
            self.tensors[s.id] = np.zeros(s.shape, np.float32)
        for s, init in zip(graph.param_syms, graph.param_inits):
            if init is None:
                t = np.zeros(s.shape, np.float32)
            elif isinstance(init, tuple) and init[0] == "random_uniform":
                t = rng.uniform(init[1], init[2], s.shape).astype(np.float32)
            else:
                t = np.zeros(int(np.prod(s.shape)), np.float32)
                d = np.asarray(init, np.float32).ravel()
                t[:d.size] = d
                t = t.reshape(s.shape)
            self.tensors[s.id] = t
        for n in graph.nodes:
            for s in n.outputs:
                self.tensors[s.id] = np.zeros(s.shape, np.float32)
        for s in list(graph.inputs) + list(graph.param_syms) + [o for n in graph.nodes for o in n.outputs]:
            if s.trainable:
                self.grads[s.id] = np.zeros(s.shape, np.float32)
        self.n_inference_nodes = 0
        out_ids = {o.id for o in graph.outputs}
        for i in range(len(graph.nodes) - 1, -1, -1):
            if any(o.id in out_ids for o in graph.nodes[i].outputs):
                self.n_inference_nodes = i + 1
                break

    def _attrs(self, n: Node):
        a = dict(n.attrs)
        if n.op == OP.POW:
            a["exponent"] = float(self.tensors[n.inputs[1].id][0])
        if n.op in (OP.FLATTEN, OP.RESHAPE, OP.SQUEEZE, OP.UNSQUEEZE):
            a["out_shape"] = n.outputs[0].shape
        a.pop("shape", None)
        a.pop("dims", None)
        return a

    def execute(self, num_nodes, inputs):
        for s, v in zip(self.g.inputs, inputs):
            self.tensors[s.id] = np.ascontiguousarray(v, np.float32).reshape(s.shape).copy()
        for n in self.g.nodes[:num_nodes]:
            t = [self.tensors[i.id] for i in n.inputs]
            if n.op == OP.CONCAT:       # dynamics.mojo:25-108
                self.tensors[n.outputs[0].id] = layout.concat_fwd(t, n.attrs["dim"])
                continue
            if n.op == OP.SPLIT:        # dynamics.mojo:111-199
                for o, piece in zip(n.outputs, layout.split_fwd(t[0], n.attrs["sections"], n.attrs["dim"])):
                    self.tensors[o.id] = piece
                continue
            if n.op == OP.POW:
                t = t[:1]
            self.tensors[n.outputs[0].id] = ops.forward_op(n.op, *t, **self._attrs(n))

    def forward(self, *inputs) -> float:
        self.execute(len(self.g.nodes), inputs)
        return float(self.tensors[self.g.loss_out.id].ravel()[0])

    def inference(self, *inputs, outputs=None):
        self.execute(self.n_inference_nodes, inputs)
        outs = self.g.outputs if outputs is None else outputs
        return [self.tensors[o.id].copy() for o in outs]

    def backward(self):
        self.grads[self.g.loss_out.id].fill(1.0)
        for n in reversed(self.g.nodes):
            t = [self.tensors[i.id] for i in n.inputs]
            if n.op == OP.CONCAT:
                shapes = [i.shape for i in n.inputs]
                for j, operand in enumerate(n.inputs):
                    if operand.trainable:
                        self.grads[operand.id] += layout.concat_bwd(self.grads[n.outputs[0].id], shapes, j, n.attrs["dim"])
                continue
            if n.op == OP.SPLIT:
                if n.inputs[0].trainable:
                    self.grads[n.inputs[0].id] += layout.split_bwd([self.grads[o.id] for o in n.outputs], n.inputs[0].shape,
                                                                   n.attrs["sections"], n.attrs["dim"])
                continue
            args = t[:1] if n.op == OP.POW else t
            while len(args) < 3:
                args = args + [None]
            for j, operand in enumerate(n.inputs):
                if not operand.trainable:
                    continue
                ops.backward_op(j, n.op, self.grads[n.outputs[0].id], args[0], args[1], args[2],
                                grad=self.grads[operand.id], **self._attrs(n))

    def zero_grads(self):
        for g in self.grads.values():
            g.fill(0.0)

    def tensor(self, s):
        return self.tensors[s.id].copy()

    def set_tensor(self, s, value):
        self.tensors[s.id] = np.ascontiguousarray(value, np.float32).reshape(s.shape).copy()

    def grad(self, s):
        return self.grads[s.id].copy()


class Adam:
    def __init__(self, model: Model, lr=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8):
        self.model, self.lr, self.beta1, self.beta2, self.eps = model, lr, beta1, beta2, epsilon
        self.iter = 0
        self.trainable = [s for s in model.g.param_syms if s.trainable]  # get_trainable_parameters
        self.m = {s.id: np.zeros(s.shape, np.float32) for s in self.trainable}
        self.v = {s.id: np.zeros(s.shape, np.float32) for s in self.trainable}
        self.grad_scale = 1.0

    def zero_grad(self):
        self.model.zero_grads()

    def step(self):
        self.iter += 1
        for s in self.trainable:
            p = self.model.tensors[s.id]
            if not p.flags["C_CONTIGUOUS"]:
                p = np.ascontiguousarray(p)
                self.model.tensors[s.id] = p
            ops.adam_step(p, self.model.grads[s.id], self.m[s.id], self.v[s.id], self.lr, self.beta1, self.beta2,
                          self.eps, self.iter, self.grad_scale)
