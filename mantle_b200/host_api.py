"""Python handles for the C++ host mirror in libmantle_host.so: Graph, Model, Adam, Trainer and
the nn builders, with the method names of the reference (mantle/autograd/graph.mojo,
mantle/nn/model.mojo, mantle/nn/optim.mojo, mantle/nn/*).  These classes only forward calls."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np

from . import _lib
from ._lib import MantleError, OP
from .runtime import Context

MTL_MAX_RANK = 8


class _Attrs(C.Structure):
    _fields_ = [("has_axis", C.c_int32), ("axis", C.c_int32), ("shape_rank", C.c_int32),
                ("shape", C.c_int64 * MTL_MAX_RANK),
                ("padding", C.c_int32 * 2), ("stride", C.c_int32 * 2), ("dilation", C.c_int32 * 2),
                ("kernel_size", C.c_int32 * 2), ("negative_slope", C.c_float),
                ("has_clip_min", C.c_int32), ("has_clip_max", C.c_int32),
                ("clip_min", C.c_float), ("clip_max", C.c_float),
                ("n_dims", C.c_int32), ("dims", C.c_int32 * MTL_MAX_RANK),
                ("n_axes", C.c_int32), ("axes", C.c_int32 * MTL_MAX_RANK),
                ("n_slice", C.c_int32), ("has_steps", C.c_int32),
                ("starts", C.c_int64 * MTL_MAX_RANK), ("ends", C.c_int64 * MTL_MAX_RANK),
                ("steps", C.c_int64 * MTL_MAX_RANK)]


def _make_attrs(attrs: dict) -> _Attrs:
    a = _Attrs()
    a.negative_slope = 0.01
    a.stride[:] = (1, 1)
    a.dilation[:] = (1, 1)
    for k, v in attrs.items():
        if v is None:
            continue
        if k == "axis":
            a.has_axis, a.axis = 1, int(v)
        elif k == "shape":
            a.shape_rank = len(v)
            a.shape[:len(v)] = [int(x) for x in v]
        elif k in ("padding", "stride", "dilation", "kernel_size"):
            getattr(a, k)[:] = [int(x) for x in v]
        elif k == "negative_slope":
            a.negative_slope = float(v)
        elif k == "min":
            a.has_clip_min, a.clip_min = 1, float(v)
        elif k == "max":
            a.has_clip_max, a.clip_max = 1, float(v)
        elif k == "dims":
            a.n_dims = len(v)
            a.dims[:len(v)] = [int(x) for x in v]
        elif k == "axes":
            a.n_axes = len(v)
            a.axes[:len(v)] = [int(x) for x in v]
        elif k in ("starts", "ends"):
            a.n_slice = len(v)
            getattr(a, k)[:len(v)] = [int(x) for x in v]
        elif k == "steps":
            a.has_steps = 1
            a.steps[:len(v)] = [int(x) for x in v]
        else:
            raise ValueError("unknown attribute %r" % k)
    return a


def _ck(rc: int):
    if rc != 0:
        raise MantleError(rc, _lib.host_lib().mtlh_last_error().decode())


class Symbol:
    def __init__(self, graph: "Graph", sid: int):
        self.graph, self.id = graph, sid
        rank, dims, tr = C.c_int32(), (C.c_int64 * MTL_MAX_RANK)(), C.c_int32()
        _ck(_lib.host_lib().mtlh_graph_symbol(graph.handle, sid, C.byref(rank), dims, C.byref(tr)))
        self.shape = tuple(dims[i] for i in range(rank.value))
        self.trainable = bool(tr.value)

    def __repr__(self):
        return "Symbol(%d, %s, trainable=%s)" % (self.id, self.shape, self.trainable)


class Graph:
    """mantle/autograd/graph.mojo: input / param / scalar / op / out / loss."""

    def __init__(self):
        self.lib = _lib.host_lib()
        h = C.c_void_p()
        _ck(self.lib.mtlh_graph_create(C.byref(h)))
        self.handle = h

    def __del__(self):
        try:
            self.lib.mtlh_graph_destroy(self.handle)
        except Exception:
            pass

    def _shape(self, shape):
        return len(shape), (C.c_int64 * len(shape))(*[int(s) for s in shape])

    def input(self, shape: Sequence[int], trainable: bool = False) -> Symbol:
        r, s = self._shape(shape)
        out = C.c_int32()
        _ck(self.lib.mtlh_graph_input(self.handle, r, s, int(trainable), C.byref(out)))
        return Symbol(self, out.value)

    def param(self, shape: Sequence[int], init=None, trainable: bool = True) -> Symbol:
        """init: None (zeros), an array of literal data, or ("random_uniform", lo, hi)."""
        r, s = self._shape(shape)
        out = C.c_int32()
        if init is None:
            _ck(self.lib.mtlh_graph_param(self.handle, r, s, 0, None, 0, C.c_float(0), C.c_float(0), int(trainable),
                                          C.byref(out)))
        elif isinstance(init, tuple) and init and init[0] == "random_uniform":
            _ck(self.lib.mtlh_graph_param(self.handle, r, s, 2, None, 0, C.c_float(init[1]), C.c_float(init[2]),
                                          int(trainable), C.byref(out)))
        else:
            data = np.ascontiguousarray(init, dtype=np.float32).ravel()
            _ck(self.lib.mtlh_graph_param(self.handle, r, s, 1, data.ctypes.data_as(C.POINTER(C.c_float)),
                                          C.c_int64(data.size), C.c_float(0), C.c_float(0), int(trainable),
                                          C.byref(out)))
        return Symbol(self, out.value)

    def scalar(self, value: float) -> Symbol:
        out = C.c_int32()
        _ck(self.lib.mtlh_graph_scalar(self.handle, C.c_float(value), C.byref(out)))
        return Symbol(self, out.value)

    def op(self, op: int, *operands, **attrs) -> Symbol:
        a = _make_attrs(attrs)
        out = C.c_int32()
        if len(operands) == 2 and isinstance(operands[1], (int, float)):
            _ck(self.lib.mtlh_graph_op_scalar(self.handle, op, operands[0].id, C.c_double(operands[1]), 0,
                                              C.byref(a), C.byref(out)))
        elif len(operands) == 2 and isinstance(operands[0], (int, float)):
            _ck(self.lib.mtlh_graph_op_scalar(self.handle, op, operands[1].id, C.c_double(operands[0]), 1,
                                              C.byref(a), C.byref(out)))
        else:
            ids = (C.c_int32 * len(operands))(*[o.id for o in operands])
            _ck(self.lib.mtlh_graph_op(self.handle, op, len(operands), ids, C.byref(a), C.byref(out)))
        return Symbol(self, out.value)

    def concat(self, *operands: Symbol, dim: int = 0) -> Symbol:
        """graph.mojo:180-193."""
        ids = (C.c_int32 * len(operands))(*[o.id for o in operands])
        out = C.c_int32()
        _ck(self.lib.mtlh_graph_concat(self.handle, len(operands), ids, int(dim), C.byref(out)))
        return Symbol(self, out.value)

    def split(self, operand: Symbol, sections: Sequence[int], dim: int = 0) -> List[Symbol]:
        """graph.mojo:200-210: one result symbol per section."""
        sec = (C.c_int64 * len(sections))(*[int(s) for s in sections])
        outs = (C.c_int32 * len(sections))()
        _ck(self.lib.mtlh_graph_split(self.handle, operand.id, len(sections), sec, int(dim), outs))
        return [Symbol(self, outs[i]) for i in range(len(sections))]

    def out(self, s: Symbol):
        _ck(self.lib.mtlh_graph_out(self.handle, s.id))

    def loss(self, s: Symbol):
        _ck(self.lib.mtlh_graph_loss(self.handle, s.id))

    def counts(self):
        n = [C.c_int32() for _ in range(4)]
        _ck(self.lib.mtlh_graph_counts(self.handle, *[C.byref(x) for x in n]))
        return {"nodes": n[0].value, "params": n[1].value, "inputs": n[2].value, "symbols": n[3].value}

    def node(self, i: int):
        op, n_in, out = C.c_int32(), C.c_int32(), C.c_int32()
        ins = (C.c_int32 * 8)()
        _ck(self.lib.mtlh_graph_node(self.handle, i, C.byref(op), C.byref(n_in), ins, C.byref(out)))
        return {"op": op.value, "inputs": [ins[j] for j in range(n_in.value)], "output": out.value}

    def params(self):
        out = []
        for i in range(self.counts()["params"]):
            sid = C.c_int32()
            _ck(self.lib.mtlh_graph_param_id(self.handle, i, C.byref(sid)))
            out.append(Symbol(self, sid.value))
        return out


class nn:
    """Graph builders, mantle/nn/{layers,activations,loss}."""

    @staticmethod
    def Linear(g: Graph, inputs: Symbol, n_outputs: int) -> Symbol:
        out = C.c_int32()
        _ck(g.lib.mtlh_nn_linear(g.handle, inputs.id, n_outputs, C.byref(out)))
        return Symbol(g, out.value)

    @staticmethod
    def Conv2d(g: Graph, inputs: Symbol, out_channels: int, kernel_size, padding=(0, 0), stride=(1, 1),
               dilation=(1, 1)) -> Symbol:
        i2 = lambda v: (C.c_int32 * 2)(*[int(x) for x in v])
        out = C.c_int32()
        _ck(g.lib.mtlh_nn_conv2d(g.handle, inputs.id, out_channels, i2(kernel_size), i2(padding), i2(stride),
                                 i2(dilation), C.byref(out)))
        return Symbol(g, out.value)

    @staticmethod
    def MaxPool2d(g: Graph, inputs: Symbol, kernel_size, stride=None, padding=(0, 0), dilation=(1, 1)) -> Symbol:
        i2 = lambda v: (C.c_int32 * 2)(*[int(x) for x in v])
        if stride is None:
            stride = (-1, -1)
        elif isinstance(stride, int):
            stride = (stride, stride)
        out = C.c_int32()
        _ck(g.lib.mtlh_nn_maxpool2d(g.handle, inputs.id, i2(kernel_size), i2(stride), i2(padding), i2(dilation),
                                    C.byref(out)))
        return Symbol(g, out.value)

    @staticmethod
    def ReLU(g: Graph, x: Symbol) -> Symbol:
        return g.op(OP.RELU, x)

    @staticmethod
    def Sigmoid(g: Graph, x: Symbol) -> Symbol:
        return g.op(OP.SIGMOID, x)

    @staticmethod
    def Tanh(g: Graph, x: Symbol) -> Symbol:
        return g.op(OP.TANH, x)

    @staticmethod
    def Softmax(g: Graph, x: Symbol, axis: int) -> Symbol:
        out = C.c_int32()
        _ck(g.lib.mtlh_nn_softmax(g.handle, x.id, axis, 0, C.byref(out)))
        return Symbol(g, out.value)

    @staticmethod
    def LogSoftmax(g: Graph, x: Symbol, axis: int) -> Symbol:
        out = C.c_int32()
        _ck(g.lib.mtlh_nn_softmax(g.handle, x.id, axis, 1, C.byref(out)))
        return Symbol(g, out.value)

    @staticmethod
    def MSELoss(g: Graph, y_pred: Symbol, y_true: Symbol) -> Symbol:
        out = C.c_int32()
        _ck(g.lib.mtlh_nn_loss(g.handle, y_pred.id, y_true.id, 0, C.byref(out)))
        return Symbol(g, out.value)

    @staticmethod
    def CrossEntropyLoss(g: Graph, y_pred: Symbol, y_true: Symbol) -> Symbol:
        out = C.c_int32()
        _ck(g.lib.mtlh_nn_loss(g.handle, y_pred.id, y_true.id, 1, C.byref(out)))
        return Symbol(g, out.value)


def _ptr_array(arrays):
    return (C.POINTER(C.c_float) * len(arrays))(*[a.ctypes.data_as(C.POINTER(C.c_float)) for a in arrays])


class Model:
    """mantle/nn/model.mojo: forward / inference / backward on a device arena."""

    def __init__(self, ctx: Context, graph: Graph, seed: int = 42):
        self.lib = _lib.host_lib()
        self.ctx, self.graph = ctx, graph
        h = C.c_void_p()
        _ck(self.lib.mtlh_model_create(C.c_void_p(ctx.handle), graph.handle, C.c_uint64(seed), C.byref(h)))
        self.handle = h

    def close(self):
        if self.handle:
            self.lib.mtlh_model_destroy(self.handle)
            self.handle = None

    def forward(self, *inputs: np.ndarray) -> float:
        arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in inputs]
        loss = C.c_float()
        _ck(self.lib.mtlh_model_forward(self.handle, len(arrs), _ptr_array(arrs), C.byref(loss)))
        return loss.value

    def inference(self, *inputs: np.ndarray, outputs: Sequence[Symbol]):
        arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in inputs]
        outs = [np.empty(s.shape, dtype=np.float32) for s in outputs]
        _ck(self.lib.mtlh_model_inference(self.handle, len(arrs), _ptr_array(arrs), len(outs), _ptr_array(outs)))
        return outs

    def backward(self):
        _ck(self.lib.mtlh_model_backward(self.handle))

    def zero_grads(self):
        _ck(self.lib.mtlh_model_zero_grads(self.handle))

    def tensor(self, s: Symbol) -> np.ndarray:
        out = np.empty(s.shape, dtype=np.float32)
        _ck(self.lib.mtlh_model_get_tensor(self.handle, s.id, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def set_tensor(self, s: Symbol, value: np.ndarray):
        v = np.ascontiguousarray(value, dtype=np.float32)
        assert v.size == int(np.prod(s.shape)), (v.shape, s.shape)
        _ck(self.lib.mtlh_model_set_tensor(self.handle, s.id, v.ctypes.data_as(C.POINTER(C.c_float))))

    def grad(self, s: Symbol) -> np.ndarray:
        out = np.empty(s.shape, dtype=np.float32)
        _ck(self.lib.mtlh_model_get_grad(self.handle, s.id, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def set_overwrite_first(self, on: bool):
        _ck(self.lib.mtlh_model_set_overwrite_first(self.handle, int(on)))

    def set_fusion(self, on: bool):
        """CONV2D+RELU forward and MAXPOOL2D+RELU backward as single launches; the CONV2D output and the
        gradient of the RELU output are then never written (every other tensor is bit-identical)."""
        _ck(self.lib.mtlh_model_set_fusion(self.handle, int(on)))

    def set_profiling(self, on: bool):
        """Per-node device timing, the counterpart of PerfMetrics (mantle/autograd/perf_utils.mojo:60-236)."""
        _ck(self.lib.mtlh_model_set_profiling(self.handle, int(on)))

    def perf_metrics(self):
        """(per-node array [n_nodes, 4]: forward ms, backward ms, forward launches, backward launches -- sums over
        the recorded passes, forward passes, backward passes)."""
        n = self.graph.counts()["nodes"]
        out = np.zeros((n, 4), np.float64)
        fp, bp = C.c_int32(), C.c_int32()
        _ck(self.lib.mtlh_model_perf_metrics(self.handle, out.ctypes.data_as(C.POINTER(C.c_double)), n, C.byref(fp), C.byref(bp)))
        return out, fp.value, bp.value

    def perf_report(self, forward: bool = True, time_format: str = "ms", print_shape: bool = False) -> str:
        """print_forward_perf_metrics / print_backward_perf_metrics as text."""
        buf = C.create_string_buffer(1 << 16)
        _ck(self.lib.mtlh_model_perf_report(self.handle, int(forward), time_format.encode(), int(print_shape), buf, len(buf)))
        return buf.value.decode()

    def n_trainable(self) -> int:
        return int(self.lib.mtlh_model_n_trainable(self.handle))


class Adam:
    """mantle/nn/optim.mojo:51-149."""

    def __init__(self, model: Model, lr=0.001, beta1=0.9, beta2=0.999, epsilon=1e-8):
        self.lib = _lib.host_lib()
        self.model = model
        h = C.c_void_p()
        _ck(self.lib.mtlh_adam_create(model.handle, C.c_float(lr), C.c_float(beta1), C.c_float(beta2),
                                      C.c_float(epsilon), C.byref(h)))
        self.handle = h

    def close(self):
        if self.handle:
            self.lib.mtlh_adam_destroy(self.handle)
            self.handle = None

    def zero_grad(self):
        _ck(self.lib.mtlh_adam_zero_grad(self.handle))

    def step(self):
        _ck(self.lib.mtlh_adam_step(self.handle))

    @property
    def iter(self) -> int:
        return self.lib.mtlh_adam_iter(self.handle)

    def _offsets(self):
        off, n = (C.c_int64 * 256)(), C.c_int32()
        _ck(self.lib.mtlh_model_trainable_offsets(self.model.handle, off, 256, C.byref(n)))
        return [off[i] for i in range(n.value)]

    def state(self, which: int) -> np.ndarray:
        """The flat momentum (which = 0) or rms (1) span, optim.mojo:142-149, as the device holds it."""
        out = np.zeros(max(self.model.n_trainable(), 1), np.float32)
        _ck(self.lib.mtlh_adam_get_state(self.handle, which, out.ctypes.data_as(C.POINTER(C.c_float))))
        return out

    def set_state(self, momentum: Sequence[np.ndarray], rms: Sequence[np.ndarray], iter: int):
        """Loads momentum / rms tensors (one per trainable parameter, in get_trainable_parameters order) and
        the step count, e.g. to continue from another implementation's state."""
        offs = self._offsets()
        for which, tensors in ((0, momentum), (1, rms)):
            flat = np.zeros(max(self.model.n_trainable(), 1), np.float32)
            for o, t in zip(offs, tensors):
                flat[o:o + t.size] = np.asarray(t, np.float32).ravel()
            _ck(self.lib.mtlh_adam_set_state(self.handle, which, flat.ctypes.data_as(C.POINTER(C.c_float))))
        _ck(self.lib.mtlh_adam_set_iter(self.handle, int(iter)))


def save_checkpoint(path: str, model: "Model", adam: "Adam" = None, iter: int = 0):
    """save_checkpoint / save_checkpoint_with_optim (mantle/serialize/checkpoint.mojo:197-300): every
    tensor of the model, and with `adam` its momentum and rms state, read back from the device arenas."""
    _ck(_lib.host_lib().mtlh_checkpoint_save(model.handle, adam.handle if adam is not None else None,
                                             str(path).encode(), int(iter)))


def load_checkpoint(path: str, model: "Model", adam: "Adam" = None):
    """load_checkpoint / load_checkpoint_with_optim (checkpoint.mojo:303-440) into the device arenas.
    Returns (iter, has_optim_state)."""
    it, has = C.c_int32(), C.c_int32()
    _ck(_lib.host_lib().mtlh_checkpoint_load(model.handle, adam.handle if adam is not None else None,
                                             str(path).encode(), C.byref(it), C.byref(has)))
    return it.value, bool(has.value)


class Trainer:
    """forward / zero_grad / backward / step as one enqueued (optionally captured) step."""

    def __init__(self, model: Model, adam: Adam, use_graph: bool = True, bucket_bytes: int = 256 * 1024,
                 fuse: bool = True):
        self.lib = _lib.host_lib()
        self.model, self.adam = model, adam
        # the training pipeline never reads per-node tensors, so CONV2D+RELU / MAXPOOL2D+RELU chains
        # run fused by default (see Model.set_fusion for what is then left unwritten)
        model.set_fusion(fuse)
        h = C.c_void_p()
        _ck(self.lib.mtlh_trainer_create(model.handle, adam.handle, int(use_graph), C.c_int64(bucket_bytes),
                                         C.byref(h)))
        self.handle = h

    def close(self):
        if self.handle:
            self.lib.mtlh_trainer_destroy(self.handle)
            self.handle = None

    def step(self, *inputs: np.ndarray) -> float:
        arrs = [np.ascontiguousarray(a, dtype=np.float32) for a in inputs]
        loss = C.c_float()
        _ck(self.lib.mtlh_trainer_step(self.handle, len(arrs), _ptr_array(arrs), C.byref(loss)))
        return loss.value

    def step_ptrs(self, ptrs: Sequence[int]) -> float:
        """Inputs given as raw host addresses (pinned buffers from mtl_host_alloc)."""
        arr = (C.POINTER(C.c_float) * len(ptrs))(*[C.cast(C.c_void_p(p), C.POINTER(C.c_float)) for p in ptrs])
        loss = C.c_float()
        _ck(self.lib.mtlh_trainer_step(self.handle, len(ptrs), arr, C.byref(loss)))
        return loss.value

    def step_async_ptrs(self, ptrs: Sequence[int], pinned_loss_ptr: int):
        arr = (C.POINTER(C.c_float) * len(ptrs))(*[C.cast(C.c_void_p(p), C.POINTER(C.c_float)) for p in ptrs])
        _ck(self.lib.mtlh_trainer_step_async(self.handle, len(ptrs), arr,
                                             C.cast(C.c_void_p(pinned_loss_ptr), C.POINTER(C.c_float))))

    def set_label_input(self, input_index: int, num_classes: int):
        """Input `input_index` ([B, num_classes] one-hot targets in the graph) is fed as B fp32 class labels;
        the one-hot rows are built on the device (examples/mnist.mojo:92-97 builds them on the host)."""
        _ck(self.lib.mtlh_trainer_set_label_input(self.handle, int(input_index), int(num_classes)))

    def set_exchange(self, on: bool):
        """Diagnostic: skip the gradient all-reduce of a data-parallel step (timing only, not a valid training run)."""
        _ck(self.lib.mtlh_trainer_set_exchange(self.handle, int(on)))

    def input_bytes_per_step(self) -> int:
        return int(self.lib.mtlh_trainer_input_bytes(self.handle))

    def graph_active(self) -> bool:
        return bool(self.lib.mtlh_trainer_graph_active(self.handle))
