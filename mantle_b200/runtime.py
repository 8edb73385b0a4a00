"""Thin object layer over the C ABI: a device context, device arrays, and the operator
dispatchers `forward_op` / `backward_op` with the argument meaning of
mantle/autograd/ops/ops.mojo:243-528.  All arithmetic happens in libmantle_cuda.so."""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import numpy as np

from . import _lib
from ._lib import OP, ConvDesc, MantleError, conv_desc

_UNARY = {OP.EXP, OP.LOG, OP.POW, OP.SIGMOID, OP.RELU, OP.TANH, OP.CLIP, OP.LEAKYRELU}
_BINARY = {OP.ADD, OP.SUB, OP.MUL, OP.DIV}
_REDUCE = {OP.SUM, OP.MEAN, OP.MAX}
_COPY = {OP.FLATTEN, OP.RESHAPE, OP.SQUEEZE, OP.UNSQUEEZE}
FLT_MAX = 3.402823466e38


def _shape_arr(shape: Sequence[int]):
    return (C.c_int64 * len(shape))(*[int(s) for s in shape])


class DeviceArray:
    """A dense row-major fp32 (or int32) tensor in device memory, owned by a Context."""

    def __init__(self, ctx: "Context", shape: Sequence[int], dtype=np.float32):
        self.ctx = ctx
        self.shape = tuple(int(s) for s in shape)
        self.dtype = np.dtype(dtype)
        self.size = int(np.prod(self.shape)) if self.shape else 1
        self.nbytes = self.size * self.dtype.itemsize
        p = C.c_void_p()
        ctx._check(ctx.lib.mtl_malloc(ctx.handle, max(self.nbytes, 4), C.byref(p)))
        self.ptr = p.value
        self._freed = False

    def numpy(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=self.dtype)
        self.ctx._check(self.ctx.lib.mtl_d2h(self.ctx.handle, out.ctypes.data, self.ptr, self.nbytes))
        return out

    def set(self, host: np.ndarray) -> "DeviceArray":
        host = np.ascontiguousarray(host, dtype=self.dtype)
        if host.size != self.size:
            raise ValueError("size mismatch: %s into %s" % (host.shape, self.shape))
        self.ctx._check(self.ctx.lib.mtl_h2d(self.ctx.handle, self.ptr, host.ctypes.data, self.nbytes))
        return self

    def zero(self) -> "DeviceArray":
        self.ctx._check(self.ctx.lib.mtl_zero(self.ctx.handle, self.ptr, self.nbytes))
        return self

    def free(self):
        if not self._freed and self.ctx.handle:
            self.ctx.lib.mtl_free(self.ctx.handle, self.ptr)
            self._freed = True

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Context:
    """One CUDA device + stream (mtl_ctx)."""

    def __init__(self, device: int = 0, math_mode: Optional[int] = None):
        self.lib = _lib.cuda_lib()
        h = C.c_void_p()
        rc = self.lib.mtl_ctx_create(device, C.byref(h))
        if rc != 0:
            raise MantleError(rc, "mtl_ctx_create(device=%d) failed: no usable CUDA device "
                                  "(this backend has no CPU path)" % device)
        self.handle = h.value
        self.device = device
        if math_mode is not None:
            self.set_math_mode(math_mode)

    def _check(self, rc: int):
        if rc != 0:
            raise MantleError(rc, self.lib.mtl_last_error(self.handle).decode())

    def close(self):
        if self.handle:
            self.lib.mtl_ctx_destroy(self.handle)
            self.handle = None

    def set_math_mode(self, mode: int):
        self._check(self.lib.mtl_ctx_set_math_mode(self.handle, mode))

    def math_mode(self) -> int:
        return self.lib.mtl_ctx_math_mode(self.handle)

    def sync(self):
        self._check(self.lib.mtl_sync(self.handle))

    def launch_count(self) -> int:
        return int(self.lib.mtl_launch_count(self.handle))

    def conv_split_tiles(self) -> int:
        return int(self.lib.mtl_conv_split_tiles(self.handle))

    def device_status(self) -> int:
        s = C.c_int32()
        self._check(self.lib.mtl_device_status(self.handle, C.byref(s)))
        return s.value

    def reserve_workspace(self, nbytes: int):
        self._check(self.lib.mtl_ctx_reserve_workspace(self.handle, nbytes))

    # ---- arrays --------------------------------------------------------------------------
    def empty(self, shape, dtype=np.float32) -> DeviceArray:
        return DeviceArray(self, shape, dtype)

    def zeros(self, shape, dtype=np.float32) -> DeviceArray:
        return DeviceArray(self, shape, dtype).zero()

    def array(self, host: np.ndarray, dtype=np.float32) -> DeviceArray:
        host = np.asarray(host, dtype=dtype)
        return DeviceArray(self, host.shape, dtype).set(host)

    # ---- timing --------------------------------------------------------------------------
    def timer_start(self, slot: int = 0):
        self._check(self.lib.mtl_timer_start(self.handle, slot))

    def timer_stop(self, slot: int = 0) -> None:
        self._check(self.lib.mtl_timer_stop(self.handle, slot))

    def timer_ms(self, slot: int = 0) -> float:
        ms = C.c_float()
        self._check(self.lib.mtl_timer_elapsed_ms(self.handle, slot, C.byref(ms)))
        return ms.value

    # ---- operators -----------------------------------------------------------------------
    def forward_op(self, op: int, res: DeviceArray, t1: DeviceArray, t2: DeviceArray = None,
                   t3: DeviceArray = None, **attrs):
        """forward_op[op, shapes, attrs](res, t1[, t2[, t3]]), ops.mojo:243-352."""
        L, h = self.lib, self.handle
        if op in _BINARY:
            self._check(L.mtl_binary_fwd(h, op, res.ptr, t1.ptr, t2.ptr, len(t1.shape), _shape_arr(t1.shape),
                                         len(t2.shape), _shape_arr(t2.shape)))
        elif op in _UNARY:
            p0, p1 = _unary_params(op, attrs)
            self._check(L.mtl_unary_fwd(h, op, res.ptr, t1.ptr, t1.size, p0, p1))
        elif op == OP.DOT:
            self._check(L.mtl_dot_fwd(h, res.ptr, t1.ptr, t2.ptr, t1.shape[0], t1.shape[1], t2.shape[1]))
        elif op in _REDUCE:
            self._check(L.mtl_reduce_fwd(h, op, res.ptr, t1.ptr, len(t1.shape), _shape_arr(t1.shape),
                                         attrs.get("axis", -1) if attrs.get("axis") is not None else -1))
        elif op in _COPY:
            self._check(L.mtl_copy_f32(h, res.ptr, t1.ptr, t1.size, 0))
        elif op == OP.CONV2D:
            d = _conv_desc_from(t1.shape, t2.shape, attrs)
            if attrs.get("fused_act") is not None:  # CONV2D followed by RELU in one launch
                self._check(L.mtl_conv2d_fwd_act(h, res.ptr, t1.ptr, t2.ptr, t3.ptr, C.byref(d), int(attrs["fused_act"])))
            else:
                self._check(L.mtl_conv2d_fwd(h, res.ptr, t1.ptr, t2.ptr, t3.ptr, C.byref(d)))
        elif op == OP.MAXPOOL2D:
            d = _pool_desc_from(t1.shape, attrs)
            idx = attrs.get("indices")
            self._check(L.mtl_maxpool2d_fwd(h, res.ptr, idx.ptr if idx is not None else None, t1.ptr, C.byref(d)))
        elif op == OP.FMA:
            self._check(L.mtl_fma_fwd(h, res.ptr, t1.ptr, t2.ptr, t3.ptr, t1.size))
        else:
            raise MantleError(3, "operator id %d is not on the GPU path" % op)

    def backward_op(self, tensor_id: int, op: int, ug: DeviceArray, t1: DeviceArray, t2: DeviceArray = None,
                    t3: DeviceArray = None, grad: DeviceArray = None, accumulate: bool = True, **attrs):
        """backward_op[tensor_id, op, ...](ug, t1[, t2[, t3]], grad), ops.mojo:355-528:
        grad += d(out)/d(operand tensor_id) . ug (overwrite when accumulate is False)."""
        L, h = self.lib, self.handle
        acc = 1 if accumulate else 0
        if op in _BINARY:
            self._check(L.mtl_binary_bwd(h, op, tensor_id, grad.ptr, ug.ptr, t1.ptr, t2.ptr, len(t1.shape),
                                         _shape_arr(t1.shape), len(t2.shape), _shape_arr(t2.shape), acc))
        elif op == OP.POW and tensor_id == 1:   # gradient of the [1]-shaped exponent
            self._check(L.mtl_pow_bwd_exponent(h, grad.ptr, ug.ptr, t1.ptr, t1.size, float(attrs["exponent"]), acc))
        elif op in _UNARY:
            p0, p1 = _unary_params(op, attrs)
            self._check(L.mtl_unary_bwd(h, op, grad.ptr, ug.ptr, t1.ptr, t1.size, p0, p1, acc))
        elif op == OP.DOT:
            self._check(L.mtl_dot_bwd(h, tensor_id, grad.ptr, ug.ptr, t1.ptr, t2.ptr, t1.shape[0], t1.shape[1],
                                      t2.shape[1], acc))
        elif op in _REDUCE:
            axis = attrs.get("axis")
            self._check(L.mtl_reduce_bwd(h, op, grad.ptr, ug.ptr, t1.ptr, len(t1.shape), _shape_arr(t1.shape),
                                         -1 if axis is None else axis, acc))
        elif op in _COPY:
            self._check(L.mtl_copy_f32(h, grad.ptr, ug.ptr, t1.size, acc))
        elif op == OP.CONV2D:
            d = _conv_desc_from(t1.shape, t2.shape, attrs)
            self._check(L.mtl_conv2d_bwd(h, tensor_id, grad.ptr, ug.ptr, t1.ptr, t2.ptr, C.byref(d), acc))
        elif op == OP.MAXPOOL2D:
            d = _pool_desc_from(t1.shape, attrs)
            idx = attrs.get("indices")
            if idx is not None and attrs.get("fused_act") is not None:
                # MAXPOOL2D.backward followed by the backward of the RELU that fed the pooling
                self._check(L.mtl_maxpool2d_bwd_idx_act(h, grad.ptr, ug.ptr, idx.ptr, attrs["pooled"].ptr, C.byref(d),
                                                        int(attrs["fused_act"]), acc))
            elif idx is not None:
                self._check(L.mtl_maxpool2d_bwd_idx(h, grad.ptr, ug.ptr, idx.ptr, C.byref(d), acc))
            else:
                self._check(L.mtl_maxpool2d_bwd(h, grad.ptr, ug.ptr, t1.ptr, C.byref(d), acc))
        elif op == OP.FMA:
            self._check(L.mtl_fma_bwd(h, tensor_id, grad.ptr, ug.ptr, t1.ptr, t2.ptr, t1.size, acc))
        else:
            raise MantleError(3, "operator id %d is not on the GPU path" % op)

    def adam_step(self, params, grads, m, v, n, lr, beta1, beta2, eps, t, grad_scale=1.0):
        self._check(self.lib.mtl_adam_step(self.handle, params.ptr, grads.ptr, m.ptr, v.ptr, n, lr, beta1, beta2,
                                           eps, t, grad_scale))


def _unary_params(op, attrs):
    if op == OP.POW:
        return float(attrs["exponent"]), 0.0
    if op == OP.LEAKYRELU:
        return float(attrs.get("negative_slope", 0.01)), 0.0
    if op == OP.CLIP:
        lo, hi = attrs.get("min"), attrs.get("max")
        return (-FLT_MAX if lo is None else float(lo)), (FLT_MAX if hi is None else float(hi))
    return 0.0, 0.0


def _conv_desc_from(x_shape, w_shape, attrs) -> ConvDesc:
    return conv_desc(x_shape[0], x_shape[1], x_shape[2], x_shape[3], w_shape[0], w_shape[2], w_shape[3],
                     attrs.get("padding", (0, 0)), attrs.get("stride", (1, 1)), attrs.get("dilation", (1, 1)))


def _pool_desc_from(x_shape, attrs) -> ConvDesc:
    k = attrs["kernel_size"]
    return conv_desc(x_shape[0], x_shape[1], x_shape[2], x_shape[3], 1, k[0], k[1],
                     attrs.get("padding", (0, 0)), attrs.get("stride", k), attrs.get("dilation", (1, 1)))


def conv2d_out_shape(x_shape, w_shape, padding=(0, 0), stride=(1, 1), dilation=(1, 1)):
    """get_result_shape through the library's host helper (no device needed)."""
    lib = _lib.cuda_lib()
    d = conv_desc(x_shape[0], x_shape[1], x_shape[2], x_shape[3], w_shape[0], w_shape[2], w_shape[3], padding,
                  stride, dilation)
    oh, ow = C.c_int32(), C.c_int32()
    rc = lib.mtl_conv2d_out_shape(C.byref(d), C.byref(oh), C.byref(ow))
    if rc != 0:
        raise MantleError(rc, "invalid convolution geometry")
    return oh.value, ow.value
