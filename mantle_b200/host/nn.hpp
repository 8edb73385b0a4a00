// Graph builders mirroring mantle/nn: layers, activations and losses add nodes to a Graph, they
// hold no arithmetic.  Node sequences are the reference's so that symbol ids and node counts match
// (e.g. CrossEntropyLoss is 9 nodes, tests/mojo/test_loss.mojo:102).
#pragma once

#include <cmath>

#include "graph.hpp"

namespace mantle {
namespace nn {

// initialisation bound: the reference computes q_sqrt(fan_in) (core/math_util.mojo:21-34), an
// approximate 1/sqrt; the exact value is used here and parity runs inject their own weights.
inline Param uniform_init(float fan_in) {
    Param p;
    p.kind = Param::UNIFORM;
    float bound = 1.0f / std::sqrt(fan_in);
    p.lo = -bound;
    p.hi = bound;
    return p;
}

// nn/layers/linear.mojo:25-46: W is [in, out]; DOT then ADD
inline Symbol Linear(Graph& g, const Symbol& inputs, int n_outputs) {
    Param init = uniform_init((float)inputs.shape[1]);
    Symbol weights = g.param(TensorShape{inputs.shape[1], n_outputs}, init);
    Symbol b = g.param(TensorShape{n_outputs}, init);
    Symbol res = g.op(MTL_OP_DOT, {inputs, weights});
    return g.op(MTL_OP_ADD, {res, b});
}

// nn/layers/conv.mojo:28-71
inline Symbol Conv2d(Graph& g, const Symbol& inputs, int out_channels, int kx, int ky, int px = 0, int py = 0,
                     int sx = 1, int sy = 1, int dx = 1, int dy = 1) {
    int64_t in_channels = inputs.shape[1];
    Param init = uniform_init((float)(in_channels * kx * ky));
    Symbol weights = g.param(TensorShape{out_channels, in_channels, kx, ky}, init);
    Symbol bias = g.param(TensorShape{out_channels}, init);
    Attributes a;
    a.padding[0] = px; a.padding[1] = py;
    a.stride[0] = sx; a.stride[1] = sy;
    a.dilation[0] = dx; a.dilation[1] = dy;
    return g.op(MTL_OP_CONV2D, {inputs, weights, bias}, a);
}

// nn/layers/pool.mojo:40-87: stride defaults to the kernel size
inline Symbol MaxPool2d(Graph& g, const Symbol& inputs, int kx, int ky, int sx = -1, int sy = -1, int px = 0,
                        int py = 0, int dx = 1, int dy = 1) {
    Attributes a;
    a.kernel_size[0] = kx; a.kernel_size[1] = ky;
    a.stride[0] = sx > 0 ? sx : kx; a.stride[1] = sy > 0 ? sy : ky;
    a.padding[0] = px; a.padding[1] = py;
    a.dilation[0] = dx; a.dilation[1] = dy;
    return g.op(MTL_OP_MAXPOOL2D, {inputs}, a);
}

inline Symbol ReLU(Graph& g, const Symbol& x) { return g.op(MTL_OP_RELU, {x}); }
inline Symbol Sigmoid(Graph& g, const Symbol& x) { return g.op(MTL_OP_SIGMOID, {x}); }
inline Symbol Tanh(Graph& g, const Symbol& x) { return g.op(MTL_OP_TANH, {x}); }

inline Attributes axis_attr(int axis) {
    Attributes a;
    a.axis = axis;
    return a;
}

// nn/activations.mojo:74-88
inline Symbol Softmax(Graph& g, const Symbol& input, int axis) {
    Symbol max_values = g.op(MTL_OP_MAX, {input}, axis_attr(axis));
    Symbol input_minus_max = g.op(MTL_OP_SUB, {input, max_values});
    Symbol exp_values = g.op(MTL_OP_EXP, {input_minus_max});
    Symbol sum_values = g.op(MTL_OP_SUM, {exp_values}, axis_attr(axis));
    return g.op(MTL_OP_DIV, {exp_values, sum_values});
}

// nn/activations.mojo:94-108
inline Symbol LogSoftmax(Graph& g, const Symbol& input, int axis) {
    Symbol max_values = g.op(MTL_OP_MAX, {input}, axis_attr(axis));
    Symbol input_minus_max = g.op(MTL_OP_SUB, {input, max_values});
    Symbol exp_values = g.op(MTL_OP_EXP, {input_minus_max});
    Symbol sum_values = g.op(MTL_OP_SUM, {exp_values}, axis_attr(axis));
    Symbol log_values = g.op(MTL_OP_LOG, {sum_values});
    return g.op(MTL_OP_SUB, {input_minus_max, log_values});
}

// nn/loss.mojo:25-38: note SUB(y_true, y_pred)
inline Symbol MSELoss(Graph& g, const Symbol& y_pred, const Symbol& y_true) {
    Symbol diff = g.op(MTL_OP_SUB, {y_true, y_pred});
    Symbol loss = g.op(MTL_OP_POW, diff, 2.0);
    return g.op(MTL_OP_MEAN, {loss});
}

// nn/loss.mojo:45-61
inline Symbol CrossEntropyLoss(Graph& g, const Symbol& y_pred, const Symbol& y_true) {
    Symbol log_softmax = LogSoftmax(g, y_pred, 1);
    Symbol targets_log_softmax = g.op(MTL_OP_MUL, {y_true, log_softmax});
    Symbol ret = g.op(MTL_OP_SUM, {targets_log_softmax});
    return g.op(MTL_OP_MUL, ret, -1.0 / (double)y_pred.shape[0]);
}

}  // namespace nn
}  // namespace mantle
