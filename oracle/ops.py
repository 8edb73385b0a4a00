"""numpy wrappers around the C oracle (TEST INFRASTRUCTURE ONLY) plus the reference's operator
dispatchers restated on top of them: forward_op / backward_op, mantle/autograd/ops/ops.mojo:243-528."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_LIB_PATH = _DIR / "libmantle_oracle.so"
_lib = None
FLT_MAX = 3.402823466e38


class OP:
    """OP.* ids, mantle/autograd/ops/ops.mojo:57-83."""
    ADD, SUB, MUL, DIV, EXP, LOG, POW, DOT, SUM, MEAN, MAX = range(11)
    FLATTEN, RESHAPE, SIGMOID, RELU, TANH, CONV2D, TRANSPOSE, MAXPOOL2D, FMA = range(11, 20)
    CLIP, SQUEEZE, UNSQUEEZE = 20, 21, 22
    CONCAT, SPLIT, SLICE = 23, 24, 25
    LEAKYRELU = 28


_BINARY = {OP.ADD, OP.SUB, OP.MUL, OP.DIV}
_UNARY = {OP.EXP, OP.LOG, OP.POW, OP.SIGMOID, OP.RELU, OP.TANH, OP.CLIP, OP.LEAKYRELU}
_REDUCE = {OP.SUM, OP.MEAN, OP.MAX}
_COPY = {OP.FLATTEN, OP.RESHAPE, OP.SQUEEZE, OP.UNSQUEEZE}


class _Desc(C.Structure):
    _fields_ = [("N", C.c_int32), ("C", C.c_int32), ("H", C.c_int32), ("W", C.c_int32),
                ("K", C.c_int32), ("R", C.c_int32), ("S", C.c_int32),
                ("pad", C.c_int32 * 2), ("stride", C.c_int32 * 2), ("dilation", C.c_int32 * 2)]


def build(force: bool = False) -> Path:
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < (_DIR / "mantle_oracle.c").stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "-B"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> C.CDLL:
    """The C restatement.  MANTLE_ORACLE_LIB names another build of mantle_oracle.c to load instead (the
    sanitizer run of the CPU tests points it at an ASan + UBSan build)."""
    global _lib
    if _lib is None:
        import os
        override = os.environ.get("MANTLE_ORACLE_LIB")
        if override:
            _lib = C.CDLL(override)
            return _lib
        if not _LIB_PATH.exists():
            build()
        _lib = C.CDLL(str(_LIB_PATH))
    return _lib


def set_threads(n: int) -> int:
    """Sets the number of host threads the oracle's parallel loops use; returns the count in effect."""
    lib().mo_set_threads(int(n))
    return int(lib().mo_max_threads())


def _f(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _shape(s):
    return (C.c_int64 * len(s))(*[int(x) for x in s])


def _desc(x_shape, K, R, S, padding, stride, dilation) -> _Desc:
    d = _Desc()
    d.N, d.C, d.H, d.W = [int(v) for v in x_shape]
    d.K, d.R, d.S = int(K), int(R), int(S)
    d.pad[:] = [int(v) for v in padding]
    d.stride[:] = [int(v) for v in stride]
    d.dilation[:] = [int(v) for v in dilation]
    return d


def broadcast_shapes(s1, s2):
    out = (C.c_int64 * 8)()
    r = lib().mo_broadcast_shapes(len(s1), _shape(s1), len(s2), _shape(s2), out)
    if r < 0:
        raise ValueError("shapes %s and %s cannot be broadcast together" % (s1, s2))
    return tuple(out[i] for i in range(r))


def dot(a, b):
    a, b = _f(a), _f(b)
    M, K = a.shape
    N = b.shape[1]
    res = np.empty((M, N), np.float32)
    lib().mo_dot(_p(res), _p(a), _p(b), C.c_int64(M), C.c_int64(K), C.c_int64(N))
    return res


def dot_transpose_t2(ug, b):
    ug, b = _f(ug), _f(b)
    M, N = ug.shape
    K = b.shape[0]
    res = np.empty((M, K), np.float32)
    lib().mo_dot_transpose_t2(_p(res), _p(ug), _p(b), C.c_int64(M), C.c_int64(K), C.c_int64(N))
    return res


def dot_transpose_t1(a, ug):
    a, ug = _f(a), _f(ug)
    M, K = a.shape
    N = ug.shape[1]
    res = np.empty((K, N), np.float32)
    lib().mo_dot_transpose_t1(_p(res), _p(a), _p(ug), C.c_int64(M), C.c_int64(K), C.c_int64(N))
    return res


def conv_out_shape(x_shape, R, S, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    d = _desc(x_shape, 1, R, S, padding, stride, dilation)
    oh, ow = C.c_int32(), C.c_int32()
    lib().mo_conv_out_shape(C.byref(d), C.byref(oh), C.byref(ow))
    return oh.value, ow.value


def conv2d_fwd(x, w, bias, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    x, w, bias = _f(x), _f(w), _f(bias)
    d = _desc(x.shape, w.shape[0], w.shape[2], w.shape[3], padding, stride, dilation)
    oh, ow = conv_out_shape(x.shape, w.shape[2], w.shape[3], padding, stride, dilation)
    out = np.empty((x.shape[0], w.shape[0], oh, ow), np.float32)
    lib().mo_conv2d_fwd(_p(out), _p(x), _p(w), _p(bias), C.byref(d))
    return out


def conv2d_bwd(tensor_id, ug, x, w, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    ug, x, w = _f(ug), _f(x), _f(w)
    d = _desc(x.shape, w.shape[0], w.shape[2], w.shape[3], padding, stride, dilation)
    shape = [x.shape, w.shape, (w.shape[0],)][tensor_id]
    res = np.zeros(shape, np.float32)
    lib().mo_conv2d_bwd(tensor_id, _p(res), _p(ug), _p(x), _p(w), C.byref(d))
    return res


def maxpool2d_fwd(x, kernel_size, padding=(0, 0), stride=None, dilation=(1, 1), return_indices=False):
    x = _f(x)
    stride = kernel_size if stride is None else stride
    d = _desc(x.shape, 1, kernel_size[0], kernel_size[1], padding, stride, dilation)
    oh, ow = conv_out_shape(x.shape, kernel_size[0], kernel_size[1], padding, stride, dilation)
    out = np.empty((x.shape[0], x.shape[1], oh, ow), np.float32)
    idx = np.empty(out.shape, np.int32)
    lib().mo_maxpool2d_fwd(_p(out), _p(idx), _p(x), C.byref(d))
    return (out, idx) if return_indices else out


def maxpool2d_bwd(ug, x, kernel_size, padding=(0, 0), stride=None, dilation=(1, 1)):
    ug, x = _f(ug), _f(x)
    stride = kernel_size if stride is None else stride
    d = _desc(x.shape, 1, kernel_size[0], kernel_size[1], padding, stride, dilation)
    res = np.zeros(x.shape, np.float32)
    lib().mo_maxpool2d_bwd(_p(res), _p(ug), _p(x), C.byref(d))
    return res


def binary_fwd(op, a, b):
    a, b = _f(a), _f(b)
    out = np.empty(broadcast_shapes(a.shape, b.shape), np.float32)
    rc = lib().mo_binary_fwd(op, _p(out), _p(a), _p(b), a.ndim, _shape(a.shape), b.ndim, _shape(b.shape))
    assert rc == 0
    return out


def binary_bwd(op, tensor_id, ug, a, b, grad=None):
    """grad += contribution (un-broadcast); returns grad (zeros when not given)."""
    ug, a, b = _f(ug), _f(a), _f(b)
    target = a if tensor_id == 0 else b
    grad = np.zeros(target.shape, np.float32) if grad is None else grad
    rc = lib().mo_binary_bwd(op, tensor_id, _p(grad), _p(ug), _p(a), _p(b), a.ndim, _shape(a.shape), b.ndim,
                             _shape(b.shape))
    assert rc == 0
    return grad


def unary_fwd(op, x, p0=0.0, p1=0.0):
    x = _f(x)
    out = np.empty_like(x)
    lib().mo_unary_fwd(op, _p(out), _p(x), C.c_int64(x.size), C.c_float(p0), C.c_float(p1))
    return out


def unary_bwd(op, ug, x, p0=0.0, p1=0.0, grad=None):
    ug, x = _f(ug), _f(x)
    grad = np.zeros(x.shape, np.float32) if grad is None else grad
    lib().mo_unary_bwd(op, _p(grad), _p(ug), _p(x), C.c_int64(x.size), C.c_float(p0), C.c_float(p1))
    return grad


def pow_bwd_exponent(ug, x, exponent, grad=None):
    """POW.backward[tensor_id = 1], basics.mojo:359-376: the gradient of the [1]-shaped exponent."""
    ug, x = _f(ug), _f(x)
    grad = np.zeros((1,), np.float32) if grad is None else grad
    lib().mo_pow_bwd_exponent(_p(grad), _p(ug), _p(x), C.c_int64(x.size), C.c_float(exponent))
    return grad


def _reduced_shape(shape, axis):
    if axis is None or axis < 0:
        return (1,)
    return tuple(1 if i == axis else s for i, s in enumerate(shape))


def reduce_fwd(op, x, axis=None):
    x = _f(x)
    out = np.empty(_reduced_shape(x.shape, axis), np.float32)
    lib().mo_reduce_fwd(op, _p(out), _p(x), x.ndim, _shape(x.shape), -1 if axis is None else axis)
    return out


def reduce_bwd(op, ug, x, axis=None, grad=None):
    ug, x = _f(ug), _f(x)
    grad = np.zeros(x.shape, np.float32) if grad is None else grad
    lib().mo_reduce_bwd(op, _p(grad), _p(ug), _p(x), x.ndim, _shape(x.shape), -1 if axis is None else axis)
    return grad


def one_hot(labels, num_classes):
    """examples/mnist.mojo:92-97: labels_one_hot[b * C + Int(labels[b])] = 1.0 on a zero tensor (fp32 labels,
    truncated toward zero); rows whose label falls outside [0, C) stay zero here."""
    lab = np.asarray(labels, np.float32).ravel()
    out = np.zeros((lab.size, int(num_classes)), np.float32)
    for b, v in enumerate(lab):
        c = int(v)
        if 0 <= c < num_classes:
            out[b, c] = 1.0
    return out


def adam_step(params, grads, m, v, lr, beta1, beta2, eps, it, grad_scale=1.0):
    """In place on float32 contiguous arrays."""
    for a in (params, grads, m, v):
        assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    lib().mo_adam_step(_p(params), _p(grads), _p(m), _p(v), C.c_int64(params.size), C.c_float(lr), C.c_float(beta1),
                       C.c_float(beta2), C.c_float(eps), int(it), C.c_float(grad_scale))


def _unary_params(op, attrs):
    if op == OP.POW:
        return float(attrs["exponent"]), 0.0
    if op == OP.LEAKYRELU:
        return float(attrs.get("negative_slope", 0.01)), 0.0
    if op == OP.CLIP:
        lo, hi = attrs.get("min"), attrs.get("max")
        return (-FLT_MAX if lo is None else float(lo)), (FLT_MAX if hi is None else float(hi))
    return 0.0, 0.0


def forward_op(op, t1, t2=None, t3=None, **attrs):
    """forward_op, ops.mojo:243-352; returns the result tensor."""
    if op in _BINARY:
        return binary_fwd(op, t1, t2)
    if op in _UNARY:
        p0, p1 = _unary_params(op, attrs)
        return unary_fwd(op, t1, p0, p1)
    if op == OP.DOT:
        return dot(t1, t2)
    if op in _REDUCE:
        return reduce_fwd(op, t1, attrs.get("axis"))
    if op in _COPY:
        return _f(t1).reshape(attrs["out_shape"]).copy()
    if op == OP.CONV2D:
        return conv2d_fwd(t1, t2, t3, attrs.get("padding", (0, 0)), attrs.get("stride", (1, 1)),
                          attrs.get("dilation", (1, 1)))
    if op == OP.MAXPOOL2D:
        return maxpool2d_fwd(t1, attrs["kernel_size"], attrs.get("padding", (0, 0)), attrs.get("stride"),
                             attrs.get("dilation", (1, 1)))
    if op == OP.FMA:
        return (_f(t1) * _f(t2) + _f(t3)).astype(np.float32)  # fma in the reference; tolerance-compared
    if op == OP.TRANSPOSE:
        from . import layout
        return layout.transpose_fwd(_f(t1), attrs.get("axes"))
    if op == OP.SLICE:
        from . import layout
        return layout.slice_fwd(_f(t1), attrs["starts"], attrs["ends"], attrs.get("steps"), attrs.get("axes"))
    raise NotImplementedError(op)


def backward_op(tensor_id, op, ug, t1, t2=None, t3=None, grad=None, **attrs):
    """backward_op, ops.mojo:355-528: grad += local gradient; returns grad."""
    if op in _BINARY:
        return binary_bwd(op, tensor_id, ug, t1, t2, grad)
    if op == OP.POW and tensor_id == 1:
        return pow_bwd_exponent(ug, t1, float(attrs["exponent"]), grad)
    if op in _UNARY:
        p0, p1 = _unary_params(op, attrs)
        return unary_bwd(op, ug, t1, p0, p1, grad)
    if op == OP.DOT:
        res = dot_transpose_t2(ug, t2) if tensor_id == 0 else dot_transpose_t1(t1, ug)
    elif op in _REDUCE:
        return reduce_bwd(op, ug, t1, attrs.get("axis"), grad)
    elif op in _COPY:
        res = _f(ug).reshape(np.shape(t1)).copy()
    elif op == OP.CONV2D:
        res = conv2d_bwd(tensor_id, ug, t1, t2, attrs.get("padding", (0, 0)), attrs.get("stride", (1, 1)),
                         attrs.get("dilation", (1, 1)))
    elif op == OP.MAXPOOL2D:
        res = maxpool2d_bwd(ug, t1, attrs["kernel_size"], attrs.get("padding", (0, 0)), attrs.get("stride"),
                            attrs.get("dilation", (1, 1)))
    elif op == OP.FMA:
        res = [_f(ug) * _f(t2), _f(ug) * _f(t1), _f(ug)][tensor_id]
    elif op == OP.TRANSPOSE:
        from . import layout
        res = layout.transpose_bwd(ug, np.shape(t1), attrs.get("axes"))
    elif op == OP.SLICE:
        from . import layout
        res = layout.slice_bwd(ug, np.shape(t1), attrs["starts"], attrs["ends"], attrs.get("steps"), attrs.get("axes"))
    else:
        raise NotImplementedError(op)
    if grad is None:
        return res.astype(np.float32)
    grad += res  # accumulate_grad, tensorutils.mojo:443-451
    return grad
