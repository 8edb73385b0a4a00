"""CPU oracle for the CUDA backend -- TEST INFRASTRUCTURE ONLY.

numpy-facing wrappers around oracle/libmantle_oracle.so (a plain-C restatement of Mantle's operator
kernels, see mantle_oracle.c) and a restatement of Mantle's graph builder / executor / Adam
(mantle/autograd/graph.mojo, mantle/nn/model.mojo, mantle/nn/optim.mojo) that runs on it.
Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this package; the
mantle_b200 package never does."""
from .ops import (OP, lib, build, set_threads, dot, dot_transpose_t1, dot_transpose_t2, conv_out_shape, conv2d_fwd, conv2d_bwd,
                  maxpool2d_fwd, maxpool2d_bwd, binary_fwd, binary_bwd, unary_fwd, unary_bwd, pow_bwd_exponent, reduce_fwd, reduce_bwd,
                  adam_step, one_hot, broadcast_shapes, forward_op, backward_op)
from .model import Graph, Model, Adam, nn, Symbol
from . import checkpoint
from . import layout
