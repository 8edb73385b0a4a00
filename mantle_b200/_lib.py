"""ctypes bindings of libmantle_cuda.so: one Python function per entry point of
include/mantle_cuda.h.  Loading fails loudly when the library has not been built; there is no
fallback implementation."""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
CUDA_LIB_PATH = _PKG / "lib" / "libmantle_cuda.so"
HOST_LIB_PATH = _PKG / "lib" / "libmantle_host.so"

MTL_MAX_RANK = 8
MTL_DP_ID_BYTES = 128

STATUS_NAMES = {0: "MTL_OK", 1: "MTL_ERR_INVALID", 2: "MTL_ERR_CUDA", 3: "MTL_ERR_UNSUPPORTED",
                4: "MTL_ERR_NOMEM", 5: "MTL_ERR_TIMEOUT", 6: "MTL_ERR_COMM"}

MATH_FP32, MATH_TF32, MATH_TF32X3 = 0, 1, 2


class OP:
    """OP.* ids, mantle/autograd/ops/ops.mojo:57-83."""
    ADD, SUB, MUL, DIV, EXP, LOG, POW, DOT, SUM, MEAN, MAX = range(11)
    FLATTEN, RESHAPE, SIGMOID, RELU, TANH, CONV2D, TRANSPOSE, MAXPOOL2D, FMA = range(11, 20)
    CLIP, SQUEEZE, UNSQUEEZE = 20, 21, 22
    CONCAT, SPLIT, SLICE = 23, 24, 25
    LEAKYRELU = 28


class ConvDesc(C.Structure):
    _fields_ = [("N", C.c_int32), ("C", C.c_int32), ("H", C.c_int32), ("W", C.c_int32),
                ("K", C.c_int32), ("R", C.c_int32), ("S", C.c_int32),
                ("pad", C.c_int32 * 2), ("stride", C.c_int32 * 2), ("dilation", C.c_int32 * 2)]


def conv_desc(N, Cc, H, W, K, R, S, pad=(0, 0), stride=(1, 1), dilation=(1, 1)) -> ConvDesc:
    d = ConvDesc()
    d.N, d.C, d.H, d.W, d.K, d.R, d.S = N, Cc, H, W, K, R, S
    d.pad[:] = pad
    d.stride[:] = stride
    d.dilation[:] = dilation
    return d


class SliceDesc(C.Structure):
    _fields_ = [("n", C.c_int32), ("axes", C.c_int32 * 8), ("starts", C.c_int64 * 8), ("ends", C.c_int64 * 8),
                ("steps", C.c_int64 * 8)]


def slice_desc(starts, ends, steps=None, axes=None) -> SliceDesc:
    """The SLICE attributes of the reference: one entry per sliced axis; `axes` defaults to 0, 1, ..."""
    d = SliceDesc()
    d.n = len(starts)
    for i in range(d.n):
        d.starts[i], d.ends[i] = starts[i], ends[i]
        d.steps[i] = 1 if steps is None else steps[i]
        d.axes[i] = -1 if axes is None else axes[i]
    return d


class MantleError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__("%s: %s" % (STATUS_NAMES.get(code, code), message))
        self.code = code


_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int32, C.c_int64, C.c_float
_pi64 = C.POINTER(C.c_int64)
_pdesc = C.POINTER(ConvDesc)
_pslice = C.POINTER(SliceDesc)
_pi32 = C.POINTER(C.c_int32)
_ppf = C.POINTER(C.c_void_p)

# name -> (restype, argtypes); every symbol declared in include/mantle_cuda.h
SIGNATURES = {
    "mtl_ctx_create": (_i32, [_i32, C.POINTER(_vp)]),
    "mtl_ctx_destroy": (_i32, [_vp]),
    "mtl_ctx_set_stream": (_i32, [_vp, _vp]),
    "mtl_ctx_stream": (_vp, [_vp]),
    "mtl_ctx_set_math_mode": (_i32, [_vp, _i32]),
    "mtl_ctx_math_mode": (_i32, [_vp]),
    "mtl_ctx_reserve_workspace": (_i32, [_vp, C.c_size_t]),
    "mtl_ctx_workspace_info": (_i32, [_vp, C.POINTER(C.c_size_t), C.POINTER(_vp), C.POINTER(_i32), C.POINTER(_i32)]),
    "mtl_sync": (_i32, [_vp]),
    "mtl_last_error": (C.c_char_p, [_vp]),
    "mtl_launch_count": (_i64, [_vp]),
    "mtl_conv_split_tiles": (_i64, [_vp]),
    "mtl_device_status": (_i32, [_vp, C.POINTER(_i32)]),
    "mtl_version": (C.c_char_p, []),
    "mtl_selftest_bounded_wait": (_i32, [_vp, _i32, C.POINTER(_i32)]),
    "mtl_malloc": (_i32, [_vp, C.c_size_t, C.POINTER(_vp)]),
    "mtl_free": (_i32, [_vp, _vp]),
    "mtl_debug_check": (_i32, [_vp]),
    "mtl_h2d": (_i32, [_vp, _vp, _vp, C.c_size_t]),
    "mtl_d2h": (_i32, [_vp, _vp, _vp, C.c_size_t]),
    "mtl_h2d_async": (_i32, [_vp, _vp, _vp, C.c_size_t]),
    "mtl_d2h_async": (_i32, [_vp, _vp, _vp, C.c_size_t]),
    "mtl_host_alloc": (_i32, [_vp, C.c_size_t, C.POINTER(_vp)]),
    "mtl_host_free": (_i32, [_vp, _vp]),
    "mtl_zero": (_i32, [_vp, _vp, C.c_size_t]),
    "mtl_fill_f32": (_i32, [_vp, _vp, _i64, _f32]),
    "mtl_one_hot_f32": (_i32, [_vp, _vp, _vp, _i64, _i64]),
    "mtl_copy_f32": (_i32, [_vp, _vp, _vp, _i64, _i32]),
    "mtl_dot_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _i64]),
    "mtl_dot_bwd": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32]),
    "mtl_linear_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64]),
    "mtl_linear_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _i32, _i32]),
    "mtl_conv2d_out_shape": (_i32, [_pdesc, C.POINTER(_i32), C.POINTER(_i32)]),
    "mtl_conv2d_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _pdesc]),
    "mtl_conv2d_bwd": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _pdesc, _i32]),
    "mtl_maxpool2d_fwd": (_i32, [_vp, _vp, _vp, _vp, _pdesc]),
    "mtl_maxpool2d_bwd": (_i32, [_vp, _vp, _vp, _vp, _pdesc, _i32]),
    "mtl_maxpool2d_bwd_idx": (_i32, [_vp, _vp, _vp, _vp, _pdesc, _i32]),
    "mtl_conv2d_bwd_fused": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _pdesc, _i32, _i32, _i32]),
    "mtl_stage_h2d": (_i32, [_vp, _i32, _vp, _vp, C.c_size_t]),
    "mtl_stage_acquire": (_i32, [_vp, _i32]),
    "mtl_stage_release": (_i32, [_vp, _i32]),
    "mtl_conv2d_fwd_act_pool": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _pdesc, _i32, _pdesc]),
    "mtl_conv2d_bwd_pooled": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _pdesc, _i32, _pdesc, _i32, _i32, _i32]),
    "mtl_conv2d_fwd_act_pool_cl": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _pdesc, _i32, _pdesc]),
    "mtl_conv2d_bwd_fused_cl": (_i32, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _pdesc, _i32, _i32, _i32]),
    "mtl_conv2d_fwd_act": (_i32, [_vp, _vp, _vp, _vp, _vp, _pdesc, _i32]),
    "mtl_maxpool2d_bwd_idx_act": (_i32, [_vp, _vp, _vp, _vp, _vp, _pdesc, _i32, _i32]),
    "mtl_transpose_fwd": (_i32, [_vp, _vp, _vp, _i32, _pi64, _pi32]),
    "mtl_transpose_bwd": (_i32, [_vp, _vp, _vp, _i32, _pi64, _pi32, _i32]),
    "mtl_slice_out_shape": (_i32, [_i32, _pi64, _pslice, _pi64]),
    "mtl_slice_fwd": (_i32, [_vp, _vp, _vp, _i32, _pi64, _pslice]),
    "mtl_slice_bwd": (_i32, [_vp, _vp, _vp, _i32, _pi64, _pslice, _i32]),
    "mtl_concat_fwd": (_i32, [_vp, _vp, _ppf, _i32, _i32, _pi64, _i32]),
    "mtl_concat_bwd": (_i32, [_vp, _vp, _vp, _i32, _i32, _i32, _pi64, _i32, _i32]),
    "mtl_split_fwd": (_i32, [_vp, _ppf, _vp, _i32, _i32, _pi64, _pi64, _i32]),
    "mtl_split_bwd": (_i32, [_vp, _vp, _ppf, _i32, _i32, _pi64, _pi64, _i32, _i32]),
    "mtl_binary_fwd": (_i32, [_vp, _i32, _vp, _vp, _vp, _i32, _pi64, _i32, _pi64]),
    "mtl_binary_bwd": (_i32, [_vp, _i32, _i32, _vp, _vp, _vp, _vp, _i32, _pi64, _i32, _pi64, _i32]),
    "mtl_unary_fwd": (_i32, [_vp, _i32, _vp, _vp, _i64, _f32, _f32]),
    "mtl_unary_bwd": (_i32, [_vp, _i32, _vp, _vp, _vp, _i64, _f32, _f32, _i32]),
    "mtl_pow_bwd_exponent": (_i32, [_vp, _vp, _vp, _vp, _i64, _f32, _i32]),
    "mtl_fma_fwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64]),
    "mtl_fma_bwd": (_i32, [_vp, _i32, _vp, _vp, _vp, _vp, _i64, _i32]),
    "mtl_reduce_fwd": (_i32, [_vp, _i32, _vp, _vp, _i32, _pi64, _i32]),
    "mtl_reduce_bwd": (_i32, [_vp, _i32, _vp, _vp, _vp, _i32, _pi64, _i32, _i32]),
    "mtl_reduce_all_static": (_i32, [_vp, _i32, _vp, _vp, _i64]),
    "mtl_cross_entropy_fwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _f32]),
    "mtl_cross_entropy_bwd": (_i32, [_vp, _vp, _vp, _vp, _i64, _i64, _f32, _i32]),
    "mtl_cross_entropy_fwd_grad": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32]),
    "mtl_adam_step": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _f32, _f32, _f32, _f32, _i32, _f32]),
    "mtl_adam_step_dev": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _f32, _f32, _f32, _f32, _vp, _f32]),
    "mtl_graph_begin": (_i32, [_vp]),
    "mtl_graph_end": (_i32, [_vp, C.POINTER(_vp)]),
    "mtl_graph_launch": (_i32, [_vp, _vp]),
    "mtl_graph_destroy": (_i32, [_vp, _vp]),
    "mtl_timer_start": (_i32, [_vp, _i32]),
    "mtl_timer_stop": (_i32, [_vp, _i32]),
    "mtl_timer_elapsed_ms": (_i32, [_vp, _i32, C.POINTER(_f32)]),
    "mtl_prof_enable": (_i32, [_vp, _i32]),
    "mtl_prof_reset": (_i32, [_vp]),
    "mtl_prof_get": (_i32, [_vp, _i32, C.POINTER(_f32), C.POINTER(_i32)]),
    "mtl_prof_range_begin": (_i32, [_vp, _i32]),
    "mtl_prof_range_end": (_i32, [_vp]),
    "mtl_prof_range_count": (_i32, [_vp, C.POINTER(_i32)]),
    "mtl_prof_range_get": (_i32, [_vp, _i32, C.POINTER(_i32), C.POINTER(_f32), C.POINTER(_i32)]),
    "mtl_prof_dump": (_i32, [_vp, C.c_char_p]),
    "mtl_dp_get_unique_id": (_i32, [C.POINTER(C.c_uint8)]),
    "mtl_dp_init": (_i32, [_vp, C.POINTER(C.c_uint8), _i32, _i32]),
    "mtl_dp_probe": (_i32, [C.POINTER(C.c_uint8), _i32, _i32, _i32]),
    "mtl_dp_status": (_i32, [_vp]),
    "mtl_dp_allreduce_async": (_i32, [_vp, _vp, _i64]),
    "mtl_dp_allreduce_tail": (_i32, [_vp, _vp, _i64]),
    "mtl_dp_tail_exchange_enabled": (_i32, [_vp]),
    "mtl_selftest_tail_exchange": (_i32, [_vp, _vp, _i32, _i32, _i32, _i32, _i32]),
    "mtl_set_grads_ready_hook": (_i32, [_vp, _vp, _vp]),
    "mtl_dp_wait": (_i32, [_vp]),
    "mtl_dp_broadcast": (_i32, [_vp, _vp, _i64, _i32]),
    "mtl_dp_destroy": (_i32, [_vp]),
    "mtl_dp_world_size": (_i32, [_vp]),
}

_cuda = None
_host = None


def cuda_lib() -> C.CDLL:
    """Loads libmantle_cuda.so and types every entry point."""
    global _cuda
    if _cuda is None:
        if not CUDA_LIB_PATH.exists():
            raise ImportError("%s is missing: build it with `python -m mantle_b200.build` "
                              "(there is no CPU fallback)" % CUDA_LIB_PATH)
        lib = C.CDLL(str(CUDA_LIB_PATH), mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        _cuda = lib
    return _cuda


def host_lib() -> C.CDLL:
    global _host
    if _host is None:
        cuda_lib()
        import os
        path = Path(os.environ.get("MANTLE_HOST_LIB") or HOST_LIB_PATH)   # another build of mantle_b200/host (sanitizer runs)
        if not path.exists():
            raise ImportError("%s is missing: build it with `python -m mantle_b200.build`" % path)
        _host = C.CDLL(str(path))
        _host.mtlh_last_error.restype = C.c_char_p
        _host.mtlh_model_n_trainable.restype = C.c_int64
        _host.mtlh_trainer_input_bytes.restype = C.c_int64
    return _host
