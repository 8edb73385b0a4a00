"""mantle_b200 -- B200 (sm_100a) execution backend for Mantle's operator registry.

The product is `lib/libmantle_cuda.so` (C ABI in include/mantle_cuda.h) plus the C++ host mirror
of Mantle's graph executor in `lib/libmantle_host.so`.  This package only binds them for tests and
benchmarks; importing it does not touch the GPU, creating a `Context` does and fails loudly when
the library or a CUDA device is missing."""
from ._lib import MATH_FP32, MATH_TF32, MATH_TF32X3, OP, ConvDesc, MantleError, SliceDesc, conv_desc, slice_desc, cuda_lib, host_lib
from .runtime import Context, DeviceArray, conv2d_out_shape

__all__ = ["MATH_FP32", "MATH_TF32", "MATH_TF32X3", "OP", "ConvDesc", "MantleError", "SliceDesc", "conv_desc", "slice_desc", "cuda_lib",
           "host_lib", "Context", "DeviceArray", "conv2d_out_shape"]
