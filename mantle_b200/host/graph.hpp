// Host-side mirror of Mantle's static graph IR: Symbol, Attribute set, Node, Graph.
// Follows mantle/autograd/{symbol,node,attributes,graph}.mojo; result shapes follow
// static_result_shape in mantle/autograd/ops/ops.mojo:104-218.
#pragma once

#include <cstdint>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

#include "mantle_cuda.h"

namespace mantle {

struct TensorShape {
    int rank = 0;
    int64_t dims[MTL_MAX_RANK] = {0};
    TensorShape() = default;
    TensorShape(std::initializer_list<int64_t> l) {
        if (l.size() > MTL_MAX_RANK) throw std::invalid_argument("rank above 8");
        for (auto v : l) dims[rank++] = v;
    }
    TensorShape(int r, const int64_t* d) : rank(r) {
        if (r < 0 || r > MTL_MAX_RANK) throw std::invalid_argument("rank above 8");
        for (int i = 0; i < r; ++i) dims[i] = d[i];
    }
    int64_t num_elements() const {
        int64_t n = 1;
        for (int i = 0; i < rank; ++i) n *= dims[i];
        return n;
    }
    int64_t operator[](int i) const { return dims[i < 0 ? rank + i : i]; }
    bool operator==(const TensorShape& o) const {
        if (rank != o.rank) return false;
        for (int i = 0; i < rank; ++i)
            if (dims[i] != o.dims[i]) return false;
        return true;
    }
    bool is_scalar() const { return rank == 1 && dims[0] == 1; }
};

// symbol.mojo:61 -- a value in the graph: creation-order id, shape, trainable flag
struct Symbol {
    int id = -1;
    TensorShape shape;
    bool trainable = false;
};

// The attributes the operators on this path read (attributes.mojo:70-111 stores them by name).
struct Attributes {
    std::optional<int> axis;                 // SUM / MEAN / MAX
    std::optional<TensorShape> shape;        // RESHAPE
    int padding[2] = {0, 0};                 // CONV2D / MAXPOOL2D
    int stride[2] = {1, 1};
    int dilation[2] = {1, 1};
    int kernel_size[2] = {0, 0};             // MAXPOOL2D
    float negative_slope = 0.01f;            // LEAKYRELU
    std::optional<float> clip_min, clip_max; // CLIP
    std::vector<int> dims;                   // SQUEEZE / UNSQUEEZE
    std::vector<int> axes;                   // TRANSPOSE (empty = reversed), SLICE (empty = 0, 1, ...)
    std::vector<int64_t> starts, ends, steps;  // SLICE (steps empty = all 1)
    int cat_dim = 0;                         // CONCAT / SPLIT: the axis
    std::vector<int64_t> sections;           // SPLIT: extents of the pieces along that axis
};

struct Node {
    int op = -1;  // OP.* id
    std::vector<Symbol> inputs;
    std::vector<Symbol> outputs;
    Attributes attrs;
};

// params.mojo:201 -- how a parameter gets its first value
struct Param {
    enum Kind { ZERO, DATA, UNIFORM } kind = ZERO;
    std::vector<float> data;
    float lo = 0.0f, hi = 0.0f;
};

struct Graph {
    std::vector<Symbol> inputs;
    std::vector<Symbol> params;        // ParamDict.symbols
    std::vector<Param> param_values;   // ParamDict.values
    std::vector<Node> nodes;
    std::vector<Symbol> outputs;
    std::optional<Symbol> loss_out;
    int symbol_count = 0;

    // graph.mojo:64-83
    Symbol create_symbol(const TensorShape& shape, const Param* data, bool trainable, bool is_input) {
        Symbol s{symbol_count++, shape, trainable};
        if (is_input) {
            inputs.push_back(s);
        } else {
            params.push_back(s);
            param_values.push_back(data ? *data : Param{});
        }
        return s;
    }
    Symbol input(const TensorShape& shape, bool trainable = false) { return create_symbol(shape, nullptr, trainable, true); }
    Symbol param(const TensorShape& shape, const Param& init, bool trainable = true) {
        return create_symbol(shape, &init, trainable, false);
    }
    Symbol param(const TensorShape& shape, bool trainable = true) { return create_symbol(shape, nullptr, trainable, false); }
    Symbol scalar(float value) {  // graph.mojo:96-97
        Param p;
        p.kind = Param::DATA;
        p.data = {value};
        return create_symbol(TensorShape{1}, &p, false, false);
    }
    void out(const Symbol& s) { outputs.push_back(s); }
    void loss(const Symbol& s) { loss_out = s; }

    static bool result_trainable(const std::vector<Symbol>& operands) {  // graph.mojo:213-217
        for (auto& o : operands)
            if (o.trainable) return true;
        return false;
    }

    // graph.mojo:110-129
    Symbol op(int op_id, const std::vector<Symbol>& operands, const Attributes& attrs = Attributes()) {
        TensorShape rs = static_result_shape(op_id, operands, attrs);
        Symbol res{symbol_count++, rs, result_trainable(operands)};
        Node n;
        n.op = op_id;
        n.inputs = operands;
        n.outputs = {res};
        n.attrs = attrs;
        nodes.push_back(std::move(n));
        return res;
    }
    // graph.mojo:180-193 -- CONCAT: any number of operands, equal shapes except along `dim`
    Symbol concat(const std::vector<Symbol>& operands, int dim = 0) {
        if (operands.empty()) throw std::invalid_argument("CONCAT needs at least one operand");
        TensorShape rs = operands[0].shape;
        if (dim < 0 || dim >= rs.rank) throw std::invalid_argument("CONCAT dim out of range");
        for (size_t i = 1; i < operands.size(); ++i) {
            const TensorShape& s = operands[i].shape;
            if (s.rank != rs.rank) throw std::invalid_argument("CONCAT operands differ in rank");
            for (int d = 0; d < rs.rank; ++d)
                if (d != dim && s[d] != operands[0].shape[d]) throw std::invalid_argument("CONCAT operands differ outside dim");
            rs.dims[dim] += s[dim];
        }
        Symbol res{symbol_count++, rs, result_trainable(operands)};
        Node n;
        n.op = MTL_OP_CONCAT;
        n.inputs = operands;
        n.outputs = {res};
        n.attrs.cat_dim = dim;
        nodes.push_back(std::move(n));
        return res;
    }
    // graph.mojo:200-210 -- SPLIT: one operand, one result per section
    std::vector<Symbol> split(const Symbol& operand, const std::vector<int64_t>& sections, int dim = 0) {
        if (dim < 0 || dim >= operand.shape.rank) throw std::invalid_argument("SPLIT dim out of range");
        int64_t total = 0;
        for (int64_t s : sections) {
            if (s <= 0) throw std::invalid_argument("SPLIT sections must be positive");
            total += s;
        }
        if (sections.empty() || total != operand.shape[dim]) throw std::invalid_argument("SPLIT sections do not add up to the axis");
        Node n;
        n.op = MTL_OP_SPLIT;
        n.inputs = {operand};
        n.attrs.cat_dim = dim;
        n.attrs.sections = sections;
        for (int64_t s : sections) {
            TensorShape rs = operand.shape;
            rs.dims[dim] = s;
            n.outputs.push_back(Symbol{symbol_count++, rs, operand.trainable});
        }
        std::vector<Symbol> res = n.outputs;
        nodes.push_back(std::move(n));
        return res;
    }
    Symbol op(int op_id, const Symbol& a, double b, const Attributes& attrs = Attributes()) {  // graph.mojo:131-143
        return op(op_id, {a, scalar((float)b)}, attrs);
    }
    Symbol op(int op_id, double a, const Symbol& b, const Attributes& attrs = Attributes()) {  // graph.mojo:145-157
        return op(op_id, {scalar((float)a), b}, attrs);
    }

    static TensorShape broadcast_shapes(const TensorShape& s1, const TensorShape& s2);
    static TensorShape reduce_shape(const TensorShape& t, const Attributes& a);
    static void conv_out(const TensorShape& in, int R, int S, const Attributes& a, int64_t* oh, int64_t* ow);
    static TensorShape static_result_shape(int op_id, const std::vector<Symbol>& operands, const Attributes& attrs);
    static mtl_slice_desc slice_desc(const Attributes& a);
};

}  // namespace mantle
