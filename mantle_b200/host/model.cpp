// Graph shape rules, the executor and Adam on top of the C ABI (see model.hpp).
#include <exception>
#include "model.hpp"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstdio>
#include <cstring>

namespace mantle {

// ------------------------------------------------------------------ shapes -----------------

// broadcast_shapes, mantle/core/tensorutils.mojo:89-127
TensorShape Graph::broadcast_shapes(const TensorShape& s1, const TensorShape& s2) {
    int ndim = std::max(s1.rank, s2.rank);
    int diff = std::abs(s1.rank - s2.rank);
    const TensorShape& big = s1.rank > s2.rank ? s1 : s2;
    const TensorShape& small = s1.rank > s2.rank ? s2 : s1;
    TensorShape res;
    res.rank = ndim;
    for (int i = ndim - 1; i >= diff; --i) {
        int64_t a = big.dims[i], b = small.dims[i - diff];
        if (a == b) res.dims[i] = a;
        else if (a == 1 || b == 1) res.dims[i] = a * b;
        else throw Error(MTL_ERR_INVALID, "shapes cannot be broadcast together");
    }
    for (int i = diff - 1; i >= 0; --i) res.dims[i] = big.dims[i];
    return res;
}

// get_reduce_shape, tensorutils.mojo:601-619; no axis -> [1] (basics.mojo:383-391)
TensorShape Graph::reduce_shape(const TensorShape& t, const Attributes& a) {
    if (!a.axis) return TensorShape{1};
    int axis = *a.axis;
    if (axis < 0 || axis >= t.rank) throw Error(MTL_ERR_INVALID, "reduction axis out of range");
    TensorShape r = t;
    r.dims[axis] = 1;
    return r;
}

// get_result_shape, mantle/autograd/ops/conv.mojo:25-58
void Graph::conv_out(const TensorShape& in, int R, int S, const Attributes& a, int64_t* oh, int64_t* ow) {
    auto fd = [](int64_t x, int64_t y) {
        int64_t q = x / y;
        if ((x % y != 0) && ((x < 0) != (y < 0))) --q;
        return q;
    };
    *oh = fd(in[-2] + 2 * a.padding[0] - (int64_t)a.dilation[0] * (R - 1) - 1, a.stride[0]) + 1;
    *ow = fd(in[-1] + 2 * a.padding[1] - (int64_t)a.dilation[1] * (S - 1) - 1, a.stride[1]) + 1;
}

TensorShape Graph::static_result_shape(int op, const std::vector<Symbol>& o, const Attributes& a) {
    auto need = [&](size_t n) {
        if (o.size() != n) throw Error(MTL_ERR_INVALID, "wrong number of operands for operator");
    };
    switch (op) {
        case MTL_OP_ADD: case MTL_OP_SUB: case MTL_OP_MUL: case MTL_OP_DIV:
            need(2);
            return broadcast_shapes(o[0].shape, o[1].shape);
        case MTL_OP_POW:
            need(2);
            return o[0].shape;
        case MTL_OP_DOT:
            need(2);
            if (o[0].shape.rank != 2 || o[1].shape.rank != 2 || o[0].shape[1] != o[1].shape[0])
                throw Error(MTL_ERR_INVALID, "DOT needs [M,K] . [K,N]");
            return TensorShape{o[0].shape[0], o[1].shape[1]};
        case MTL_OP_EXP: case MTL_OP_LOG: case MTL_OP_SIGMOID: case MTL_OP_RELU: case MTL_OP_LEAKYRELU:
        case MTL_OP_TANH: case MTL_OP_CLIP:
            need(1);
            return o[0].shape;
        case MTL_OP_SUM: case MTL_OP_MEAN: case MTL_OP_MAX:
            need(1);
            return reduce_shape(o[0].shape, a);
        case MTL_OP_FLATTEN:
            need(1);
            return TensorShape{o[0].shape[0], o[0].shape.num_elements() / o[0].shape[0]};
        case MTL_OP_RESHAPE:
            need(1);
            if (!a.shape || a.shape->num_elements() != o[0].shape.num_elements())
                throw Error(MTL_ERR_INVALID, "RESHAPE needs a shape attribute with the same number of elements");
            return *a.shape;
        case MTL_OP_SQUEEZE: {  // mlops.mojo:302-316
            need(1);
            TensorShape r;
            for (int i = 0; i < o[0].shape.rank; ++i) {
                bool listed = std::find(a.dims.begin(), a.dims.end(), i) != a.dims.end();
                if ((a.dims.empty() && o[0].shape[i] == 1) || (listed && o[0].shape[i] == 1)) continue;
                r.dims[r.rank++] = o[0].shape[i];
            }
            return r;
        }
        case MTL_OP_UNSQUEEZE: {  // mlops.mojo:336-353
            need(1);
            int new_rank = o[0].shape.rank + (int)a.dims.size();
            if (new_rank > MTL_MAX_RANK) throw Error(MTL_ERR_INVALID, "rank above 8");
            TensorShape r;
            int j = 0;
            for (int i = 0; i < new_rank; ++i) {
                bool listed = std::find(a.dims.begin(), a.dims.end(), i) != a.dims.end() ||
                              std::find(a.dims.begin(), a.dims.end(), i - new_rank) != a.dims.end();
                r.dims[r.rank++] = listed ? 1 : o[0].shape[j++];
            }
            return r;
        }
        case MTL_OP_CONV2D: {  // conv.mojo:63-78
            need(3);
            if (o[0].shape.rank != 4 || o[1].shape.rank != 4 || o[0].shape[1] != o[1].shape[1])
                throw Error(MTL_ERR_INVALID, "CONV2D needs [N,C,H,W] and [K,C,R,S]");
            int64_t oh, ow;
            conv_out(o[0].shape, (int)o[1].shape[2], (int)o[1].shape[3], a, &oh, &ow);
            return TensorShape{o[0].shape[0], o[1].shape[0], oh, ow};
        }
        case MTL_OP_MAXPOOL2D: {  // pool.mojo:25-41
            need(1);
            if (o[0].shape.rank != 4) throw Error(MTL_ERR_INVALID, "MAXPOOL2D needs [N,C,H,W]");
            int64_t oh, ow;
            conv_out(o[0].shape, a.kernel_size[0], a.kernel_size[1], a, &oh, &ow);
            return TensorShape{o[0].shape[0], o[0].shape[1], oh, ow};
        }
        case MTL_OP_FMA:
            need(3);
            return o[0].shape;
        case MTL_OP_TRANSPOSE: {  // basics.mojo:618-637
            need(1);
            const int rank = o[0].shape.rank;
            if (!a.axes.empty() && (int)a.axes.size() != rank)
                throw Error(MTL_ERR_INVALID, "TRANSPOSE axes must name every axis once");
            TensorShape r;
            r.rank = rank;
            for (int i = 0; i < rank; ++i) {
                const int ax = a.axes.empty() ? rank - 1 - i : a.axes[i];
                if (ax < 0 || ax >= rank) throw Error(MTL_ERR_INVALID, "TRANSPOSE axis out of range");
                r.dims[i] = o[0].shape[ax];
            }
            return r;
        }
        case MTL_OP_SLICE: {  // mlops.mojo:420-450
            need(1);
            mtl_slice_desc d = slice_desc(a);
            TensorShape r;
            r.rank = o[0].shape.rank;
            if (mtl_slice_out_shape(o[0].shape.rank, o[0].shape.dims, &d, r.dims) != MTL_OK)
                throw Error(MTL_ERR_INVALID, "SLICE attributes do not select a non-empty part of the tensor");
            return r;
        }
        default:
            throw Error(MTL_ERR_UNSUPPORTED, "operator id " + std::to_string(op) + " is not on the GPU path");
    }
}

// SLICE attributes in the C ABI's form
mtl_slice_desc Graph::slice_desc(const Attributes& a) {
    mtl_slice_desc d;
    std::memset(&d, 0, sizeof(d));
    if (a.starts.size() != a.ends.size() || a.starts.size() > (size_t)MTL_MAX_RANK ||
        (!a.steps.empty() && a.steps.size() != a.starts.size()) || (!a.axes.empty() && a.axes.size() != a.starts.size()))
        throw Error(MTL_ERR_INVALID, "SLICE needs starts, ends (and steps, axes) of one length");
    d.n = (int32_t)a.starts.size();
    for (int i = 0; i < d.n; ++i) {
        d.starts[i] = a.starts[i];
        d.ends[i] = a.ends[i];
        d.steps[i] = a.steps.empty() ? 1 : a.steps[i];
        d.axes[i] = a.axes.empty() ? -1 : a.axes[i];
    }
    return d;
}

// ------------------------------------------------------------------ Model ------------------

namespace {
constexpr int64_t kAlign = 64;  // floats: 256-byte alignment of every tensor in the arenas
int64_t align_up(int64_t n) { return (n + kAlign - 1) / kAlign * kAlign; }

struct SplitMix {
    uint64_t s;
    explicit SplitMix(uint64_t seed) : s(seed) {}
    uint64_t next() {
        uint64_t z = (s += 0x9E3779B97F4A7C15ull);
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    float uniform(float lo, float hi) { return lo + (hi - lo) * (float)((next() >> 40) * (1.0 / 16777216.0)); }
};
}  // namespace

void Model::check(int rc, const char* what) const {
    if (rc != MTL_OK) throw Error(rc, std::string(what) + ": " + mtl_last_error(ctx_));
}

Model::Model(mtl_ctx* ctx, const Graph& g, uint64_t init_seed) : ctx_(ctx), g_(g) {
    if (!ctx) throw Error(MTL_ERR_INVALID, "null context");
    // get_trainable_parameters order (optim.mojo:27-44) first, so that the span is contiguous
    int64_t off = 0;
    for (size_t i = 0; i < g_.params.size(); ++i) {
        const Symbol& p = g_.params[i];
        if (!p.trainable) continue;
        trainable_.push_back(p);
        trainable_off_.push_back(off);
        tensor_off_[p.id] = off;
        grad_off_[p.id] = off;
        shapes_[p.id] = p.shape;
        off += align_up(p.shape.num_elements());
    }
    n_trainable_ = off;
    // RESHAPE / FLATTEN / SQUEEZE / UNSQUEEZE move no data (basics.mojo:706-756 and mlops.mojo:302-373 copy
    // element i to element i): when such a node is the ONLY reader of a node output, its result shares
    // that tensor's storage, and so do the two gradients, instead of being copied each way every step.
    // Both symbols keep their own shape and can be read by name; every value is what the copies gave.
    {
        std::map<int, int> uses, producer;
        for (size_t i = 0; i < g_.nodes.size(); ++i) {
            for (auto& s : g_.nodes[i].inputs) uses[s.id]++;
            for (auto& s : g_.nodes[i].outputs) producer[s.id] = (int)i;
        }
        alias_node_.assign(g_.nodes.size(), 0);
        for (size_t i = 0; i < g_.nodes.size(); ++i) {
            const Node& n = g_.nodes[i];
            const bool is_copy = n.op == MTL_OP_RESHAPE || n.op == MTL_OP_FLATTEN || n.op == MTL_OP_SQUEEZE || n.op == MTL_OP_UNSQUEEZE;
            if (!is_copy || n.inputs.size() != 1 || n.outputs.size() != 1) continue;
            const Symbol& in = n.inputs[0];
            const Symbol& out = n.outputs[0];
            if (!producer.count(in.id) || uses[in.id] != 1 || in.trainable != out.trainable) continue;
            if (in.shape.num_elements() != out.shape.num_elements()) continue;
            alias_of_[out.id] = in.id;
            alias_node_[i] = 1;
        }
    }
    int64_t toff = off, goff = off;
    std::map<int, bool> listed;
    auto add_tensor = [&](const Symbol& s) {
        shapes_[s.id] = s.shape;
        if (!listed[s.id]) {
            listed[s.id] = true;
            alloc_order_.push_back(s);
        }
        auto al = alias_of_.find(s.id);
        if (al != alias_of_.end() && tensor_off_.count(al->second)) {   // the producer's output was placed earlier
            tensor_off_[s.id] = tensor_off_.at(al->second);
            if (s.trainable) grad_off_[s.id] = grad_off_.at(al->second);
            return;
        }
        if (!tensor_off_.count(s.id)) {
            tensor_off_[s.id] = toff;
            toff += align_up(s.shape.num_elements());
        }
        if (s.trainable && !grad_off_.count(s.id)) {
            grad_off_[s.id] = goff;
            goff += align_up(s.shape.num_elements());
        }
    };
    // allocate_tensor_memory / allocate_grad_memory walk order (model.mojo:332-395)
    for (auto& s : g_.inputs) add_tensor(s);
    for (auto& s : g_.params) add_tensor(s);
    for (auto& n : g_.nodes)
        for (auto& s : n.outputs) add_tensor(s);
    n_tensor_floats_ = std::max<int64_t>(toff, kAlign);
    n_grad_floats_ = std::max<int64_t>(goff, kAlign);
    check(mtl_malloc(ctx_, (size_t)n_tensor_floats_ * 4, (void**)&tensors_), "tensor arena");
    check(mtl_malloc(ctx_, (size_t)n_grad_floats_ * 4, (void**)&grads_), "gradient arena");
    check(mtl_zero(ctx_, tensors_, (size_t)n_tensor_floats_ * 4), "zero tensors");
    check(mtl_zero(ctx_, grads_, (size_t)n_grad_floats_ * 4), "zero grads");

    // parameter initialisation (model.mojo:337-367)
    for (size_t i = 0; i < g_.params.size(); ++i) {
        const Symbol& p = g_.params[i];
        const Param& v = g_.param_values[i];
        int64_t n = p.shape.num_elements();
        if (v.kind == Param::ZERO) continue;
        std::vector<float> host((size_t)n, 0.0f);
        if (v.kind == Param::DATA) {
            for (size_t j = 0; j < v.data.size() && (int64_t)j < n; ++j) host[j] = v.data[j];
            if (p.shape.is_scalar() && !v.data.empty()) scalar_values_[p.id] = v.data[0];
        } else {
            SplitMix rng(init_seed * 0x100000001B3ull + (uint64_t)p.id);
            for (auto& x : host) x = rng.uniform(v.lo, v.hi);
        }
        check(mtl_h2d(ctx_, T(p), host.data(), (size_t)n * 4), "parameter upload");
    }

    // hidden argmax buffers for MAXPOOL2D nodes
    for (size_t i = 0; i < g_.nodes.size(); ++i) {
        if (g_.nodes[i].op != MTL_OP_MAXPOOL2D) continue;
        int32_t* idx = nullptr;
        check(mtl_malloc(ctx_, (size_t)g_.nodes[i].outputs[0].shape.num_elements() * 4, (void**)&idx), "pool indices");
        pool_idx_[(int)i] = idx;
    }

    // n_inference_nodes (model.mojo:47-59)
    n_inference_nodes_ = 0;
    for (int i = (int)g_.nodes.size() - 1; i >= 0 && !n_inference_nodes_; --i)
        for (auto& o : g_.nodes[i].outputs)
            for (auto& go : g_.outputs)
                if (go.id == o.id) n_inference_nodes_ = i + 1;
    check(mtl_sync(ctx_), "model setup");
}

Model::~Model() {
    for (auto& kv : pool_idx_) mtl_free(ctx_, kv.second);
    for (auto& kv : twins_) mtl_free(ctx_, kv.second);
    mtl_free(ctx_, tensors_);
    mtl_free(ctx_, grads_);
}

float* Model::T(const Symbol& s) const {
    auto it = tensor_off_.find(s.id);
    if (it == tensor_off_.end()) throw Error(MTL_ERR_INVALID, "unknown symbol " + std::to_string(s.id));
    return tensors_ + it->second;
}
float* Model::G(const Symbol& s) const {
    auto it = grad_off_.find(s.id);
    if (it == grad_off_.end()) throw Error(MTL_ERR_INVALID, "symbol " + std::to_string(s.id) + " has no gradient");
    return grads_ + it->second;
}

TensorShape Model::shape_of(int id) const {
    auto it = shapes_.find(id);
    if (it == shapes_.end()) throw Error(MTL_ERR_INVALID, "unknown symbol " + std::to_string(id));
    return it->second;
}

void Model::get_tensor(int id, float* out) const {
    Symbol s{id, shape_of(id), false};
    check(mtl_d2h(ctx_, out, T(s), (size_t)s.shape.num_elements() * 4), "get_tensor");
}
const float* Model::twin_of(const Symbol& s) const {
    auto v = twin_valid_.find(s.id);
    if (!fusion_ || v == twin_valid_.end() || !v->second) return nullptr;
    return twins_.at(s.id);
}

void Model::set_tensor(int id, const float* in) {
    twin_valid_[id] = false;  // a channels-last twin no longer matches
    Symbol s{id, shape_of(id), false};
    check(mtl_h2d(ctx_, T(s), in, (size_t)s.shape.num_elements() * 4), "set_tensor");
    if (s.shape.is_scalar() && scalar_values_.count(id)) scalar_values_[id] = in[0];
}
void Model::get_grad(int id, float* out) const {
    Symbol s{id, shape_of(id), true};
    check(mtl_d2h(ctx_, out, G(s), (size_t)s.shape.num_elements() * 4), "get_grad");
}

void Model::zero_grads() {
    if (!overwrite_first_) check(mtl_zero(ctx_, grads_, (size_t)n_grad_floats_ * 4), "zero_grad");
    // with overwrite_first the first writer of each buffer replaces its contents and buffers that
    // no node writes still hold the zeros they were created with
}

void Model::copy_inputs_async(const std::vector<const float*>& in) {
    if (in.empty()) return;  // keep the inputs already resident in the arena
    if (in.size() != g_.inputs.size()) throw Error(MTL_ERR_INVALID, "wrong number of inputs");
    for (size_t i = 0; i < in.size(); ++i)
        check(mtl_h2d_async(ctx_, T(g_.inputs[i]), in[i], (size_t)g_.inputs[i].shape.num_elements() * 4), "input copy");
}

float* Model::loss_device() const {
    if (!g_.loss_out) throw Error(MTL_ERR_INVALID, "no loss defined: Model.forward unavailable");
    return T(*g_.loss_out);
}

float Model::forward(const std::vector<const float*>& in) {
    if (!g_.loss_out) throw Error(MTL_ERR_INVALID, "no loss defined: Model.forward unavailable");
    if (in.size() != g_.inputs.size()) throw Error(MTL_ERR_INVALID, "wrong number of inputs");
    for (size_t i = 0; i < in.size(); ++i)
        check(mtl_h2d(ctx_, T(g_.inputs[i]), in[i], (size_t)g_.inputs[i].shape.num_elements() * 4), "input copy");
    execute((int)g_.nodes.size());
    float loss = 0.0f;
    check(mtl_d2h(ctx_, &loss, T(*g_.loss_out), 4), "loss read-back");
    return loss;
}

void Model::inference(const std::vector<const float*>& in, const std::vector<float*>& out) {
    if (!n_inference_nodes_) throw Error(MTL_ERR_INVALID, "no graph out defined: Model.inference unavailable");
    if (in.size() != g_.inputs.size() || out.size() != g_.outputs.size())
        throw Error(MTL_ERR_INVALID, "wrong number of inputs or outputs");
    for (size_t i = 0; i < in.size(); ++i)
        check(mtl_h2d(ctx_, T(g_.inputs[i]), in[i], (size_t)g_.inputs[i].shape.num_elements() * 4), "input copy");
    execute(n_inference_nodes_);
    for (size_t i = 0; i < out.size(); ++i)
        check(mtl_d2h(ctx_, out[i], T(g_.outputs[i]), (size_t)g_.outputs[i].shape.num_elements() * 4), "output copy");
}

namespace {
constexpr int32_t kBackwardTag = 1 << 20;  // profile tags: node index, plus this for the backward pass
// Brackets one node's calls as a profiling range when the model profiles.
struct NodeRange {
    mtl_ctx* ctx;
    bool on;
    NodeRange(mtl_ctx* c, bool enabled, int32_t tag) : ctx(c), on(enabled) {
        if (on) mtl_prof_range_begin(ctx, tag);
    }
    ~NodeRange() {
        if (on) mtl_prof_range_end(ctx);
    }
};
}  // namespace

void Model::execute(int num_nodes) {
    if (profiling_) ++fwd_passes_;
    for (int i = 0; i < num_nodes; ++i) {
        if (fusion_ && fwd_skip_[i]) continue;  // computed by the call at the head of its chain
        NodeRange range(ctx_, profiling_, i);
        if (fusion_ && i == ce_head_) {
            const Symbol& x = g_.nodes[i].inputs[0];
            // When the logits' gradient has no other contributor, the forward launch writes it as well and
            // the backward pass finds it there (the seed is 1 and neither logits nor targets change in between).
            if (overwrite_first_ && ce_sole_reader_) {
                check(mtl_cross_entropy_fwd_grad(ctx_, T(*g_.loss_out), G(x), T(x), T(g_.nodes[i + 6].inputs[0]), x.shape[0],
                                                 x.shape[1], scalar_values_.at(ce_scale_sym_)), "CrossEntropyLoss forward");
                ce_grad_fresh_ = true;
            } else {
                check(mtl_cross_entropy_fwd(ctx_, T(*g_.loss_out), T(x), T(g_.nodes[i + 6].inputs[0]), x.shape[0], x.shape[1],
                                            scalar_values_.at(ce_scale_sym_)), "CrossEntropyLoss forward");
            }
            continue;
        }
        forward_op(g_.nodes[i]);
    }
}

void Model::set_profiling(bool on) {
    profiling_ = on;
    fwd_passes_ = bwd_passes_ = 0;
    check(mtl_prof_reset(ctx_), "profile reset");
    check(mtl_prof_enable(ctx_, on ? 1 : 0), "profile switch");
}

std::vector<Model::NodePerf> Model::perf_metrics(int* fwd_passes, int* bwd_passes) {
    std::vector<NodePerf> out(g_.nodes.size());
    int32_t n = 0;
    check(mtl_prof_range_count(ctx_, &n), "profile read-out");
    for (int32_t r = 0; r < n; ++r) {
        int32_t tag = 0, launches = 0;
        float ms = 0.0f;
        check(mtl_prof_range_get(ctx_, r, &tag, &ms, &launches), "profile read-out");
        const bool bwd = tag >= kBackwardTag;
        const int node = bwd ? tag - kBackwardTag : tag;
        if (node < 0 || (size_t)node >= out.size()) continue;
        if (bwd) { out[node].bwd_ms += ms; out[node].bwd_launches += launches; }
        else     { out[node].fwd_ms += ms; out[node].fwd_launches += launches; }
    }
    if (fwd_passes) *fwd_passes = fwd_passes_;
    if (bwd_passes) *bwd_passes = bwd_passes_;
    return out;
}

static const char* op_name(int op) {
    switch (op) {
        case MTL_OP_ADD: return "ADD"; case MTL_OP_SUB: return "SUB"; case MTL_OP_MUL: return "MUL";
        case MTL_OP_DIV: return "DIV"; case MTL_OP_EXP: return "EXP"; case MTL_OP_LOG: return "LOG";
        case MTL_OP_POW: return "POW"; case MTL_OP_DOT: return "DOT"; case MTL_OP_SUM: return "SUM";
        case MTL_OP_MEAN: return "MEAN"; case MTL_OP_MAX: return "MAX"; case MTL_OP_FLATTEN: return "FLATTEN";
        case MTL_OP_RESHAPE: return "RESHAPE"; case MTL_OP_SIGMOID: return "SIGMOID"; case MTL_OP_RELU: return "RELU";
        case MTL_OP_TANH: return "TANH"; case MTL_OP_CONV2D: return "CONV2D"; case MTL_OP_TRANSPOSE: return "TRANSPOSE";
        case MTL_OP_MAXPOOL2D: return "MAXPOOL2D"; case MTL_OP_FMA: return "FMA"; case MTL_OP_CLIP: return "CLIP";
        case MTL_OP_SQUEEZE: return "SQUEEZE"; case MTL_OP_UNSQUEEZE: return "UNSQUEEZE"; case MTL_OP_CONCAT: return "CONCAT";
        case MTL_OP_SPLIT: return "SPLIT"; case MTL_OP_SLICE: return "SLICE"; case MTL_OP_LEAKYRELU: return "LEAKYRELU";
        default: return "?";
    }
}

std::string Model::perf_report(bool forward, const std::string& time_format, bool print_shape) {
    int fp = 0, bp = 0;
    std::vector<NodePerf> m = perf_metrics(&fp, &bp);
    const int passes = std::max(1, forward ? fp : bp);
    const double unit = time_format == "ns" ? 1e6 : time_format == "s" ? 1e-3 : 1.0;  // from milliseconds
    double total = 0;
    for (auto& v : m) total += forward ? v.fwd_ms : v.bwd_ms;
    auto fit = [](std::string s, size_t n) { s.resize(std::max(n, s.size()), ' '); return s.substr(0, n); };
    auto shape_str = [](const TensorShape& t) {
        std::string r = "<";
        for (int i = 0; i < t.rank; ++i) r += (i ? "x" : "") + std::to_string(t.dims[i]);
        return r + ">";
    };
    char buf[64];
    std::string out = forward ? "\n\nForward pass performance metrics:\n" : "\n\nBackward pass performance metrics:\n";
    out += fit("Node", 5) + "| " + fit("Operator", 15) + "| " + fit("Time [" + time_format + "]", 20) + "| " +
           fit("Percentage [%]", 20) + "| " + fit("Kernels", 8);
    if (print_shape) out += "| Shape\t <out> = OP( <in1>, <in2>, <in3> )";
    out += "\n";
    for (size_t i = 0; i < m.size(); ++i) {
        const double ms = forward ? m[i].fwd_ms : m[i].bwd_ms;
        const int64_t launches = forward ? m[i].fwd_launches : m[i].bwd_launches;
        snprintf(buf, sizeof(buf), "%.4f", ms / passes * unit);
        out += fit(std::to_string(i), 5) + "| " + fit(op_name(g_.nodes[i].op), 15) + "| " + fit(buf, 20) + "| ";
        snprintf(buf, sizeof(buf), "%.3f %%", total > 0 ? 100.0 * ms / total : 0.0);
        out += fit(buf, 20) + "| " + fit(std::to_string(launches / passes), 8);
        if (print_shape) {
            out += "| ";
            for (size_t j = 0; j < g_.nodes[i].outputs.size(); ++j) out += (j ? ", " : "") + fit(shape_str(g_.nodes[i].outputs[j].shape), 15);
            out += " = OP(";
            for (size_t j = 0; j < g_.nodes[i].inputs.size(); ++j) out += (j ? ", " : "") + fit(shape_str(g_.nodes[i].inputs[j].shape), 15);
            out += ")";
        }
        out += "\n";
    }
    snprintf(buf, sizeof(buf), "%.6f", total / passes * unit);
    out += std::string("\nTotal average ") + (forward ? "Forward" : "Backward") + " time: " + buf + " " + time_format + "\n";
    return out;
}

void Model::set_fusion(bool on) {
    const int nn = (int)g_.nodes.size();
    fusion_ = on;
    twin_valid_.clear();
    fwd_relu_of_.assign(nn, -1);
    fwd_pool_of_.assign(nn, -1);
    bwd_relu_of_.assign(nn, -1);
    bwd_pooled_of_.assign(nn, -1);
    bwd_pool_skip_.assign(nn, 0);
    fwd_skip_.assign(nn, 0);
    bwd_skip_.assign(nn, 0);
    relu_in_absent_.assign(nn, 0);
    lin_add_of_.assign(nn, -1);
    lin_dot_of_.assign(nn, -1);
    ce_head_ = -1;
    ce_sole_reader_ = false;
    ce_grad_fresh_ = false;
    if (!on) return;
    std::map<int, int> uses, producer;
    for (int i = 0; i < nn; ++i) {
        for (auto& s : g_.nodes[i].inputs) uses[s.id]++;
        for (auto& s : g_.nodes[i].outputs) producer[s.id] = i;
    }
    auto visible = [&](const Symbol& s) {  // a tensor the user can ask for by name
        for (auto& o : g_.outputs) if (o.id == s.id) return true;
        return g_.loss_out && g_.loss_out->id == s.id;
    };
    for (int j = 0; j < nn; ++j) {
        const Node& r = g_.nodes[j];
        if (r.op != MTL_OP_RELU) continue;
        const Symbol& rin = r.inputs[0];
        const Symbol& rout = r.outputs[0];
        const bool only_reader = uses[rin.id] == 1 && !visible(rin);
        auto p = producer.find(rin.id);
        if (only_reader && p != producer.end() && g_.nodes[p->second].op == MTL_OP_CONV2D && ((p->second < n_inference_nodes_) == (j < n_inference_nodes_) || n_inference_nodes_ == 0)) {
            fwd_relu_of_[p->second] = j;
            fwd_skip_[j] = 1;
            relu_in_absent_[j] = 1;
        }
        // backward: the single consumer of the RELU output is a MAXPOOL2D, and the RELU is the single
        // writer of its input's gradient (so the order of accumulation cannot change)
        if (uses[rout.id] == 1 && !visible(rout) && only_reader && rin.trainable) {
            for (int k = j + 1; k < nn; ++k) {
                const Node& q = g_.nodes[k];
                if (q.op == MTL_OP_MAXPOOL2D && q.inputs[0].id == rout.id) {
                    bwd_relu_of_[k] = j;
                    bwd_skip_[j] = 1;
                }
            }
        }
        // forward: CONV2D -> RELU -> MAXPOOL2D as one call when neither intermediate tensor is needed
        // (the pooling's backward then works from the indices and the pooled values alone)
        if (fwd_skip_[j] && uses[rout.id] == 1 && !visible(rout) && (bwd_skip_[j] || !rout.trainable)) {
            for (int k = j + 1; k < nn; ++k) {
                const Node& q = g_.nodes[k];
                if (q.op == MTL_OP_MAXPOOL2D && q.inputs[0].id == rout.id &&
                    ((k < n_inference_nodes_) == (j < n_inference_nodes_) || n_inference_nodes_ == 0)) {
                    fwd_pool_of_[p->second] = k;
                    fwd_skip_[k] = 1;
                    // backward: the layer's gradients come straight from the pooled gradient and the dense
                    // gradient of its output is never written in NCHW
                    const Node& cv = g_.nodes[p->second];
                    if (bwd_skip_[j] && bwd_relu_of_[k] == j &&
                        (cv.inputs[0].trainable || cv.inputs[1].trainable || cv.inputs[2].trainable)) {
                        bwd_pooled_of_[p->second] = k;
                        bwd_pool_skip_[k] = 1;
                    }
                    // a CONV2D reads the pooled output: keep a channels-last twin of it, written by the
                    // producing call and read by that layer's tensor-core kernels instead of their own copy
                    const Symbol& po = q.outputs[0];
                    bool feeds_conv = false;
                    for (int c2 = k + 1; c2 < nn; ++c2)
                        if (g_.nodes[c2].op == MTL_OP_CONV2D && g_.nodes[c2].inputs[0].id == po.id) feeds_conv = true;
                    if (feeds_conv && !twins_.count(po.id)) {
                        float* t = nullptr;
                        check(mtl_malloc(ctx_, (size_t)po.shape.num_elements() * 4, (void**)&t), "channels-last twin");
                        twins_[po.id] = t;
                    }
                }
            }
        }
    }
    // nn.Linear with a narrow output (linear.mojo:25-46): DOT whose only reader is an ADD of a [N] bias, N <= 16.
    // One mtl_linear_fwd / mtl_linear_bwd call covers both nodes; the DOT's own output and its gradient are
    // not materialised.
    for (int i = 0; i < nn; ++i) {
        const Node& d = g_.nodes[i];
        if (d.op != MTL_OP_DOT || d.outputs.size() != 1) continue;
        const Symbol& dout = d.outputs[0];
        if (uses[dout.id] != 1 || visible(dout) || d.inputs[1].shape[1] > 16) continue;
        for (int j = i + 1; j < nn; ++j) {
            const Node& a = g_.nodes[j];
            if (a.op != MTL_OP_ADD || a.inputs.size() != 2 || a.inputs[0].id != dout.id) continue;
            const Symbol& bias = a.inputs[1];
            const bool row_bias = (bias.shape.rank == 1 && bias.shape[0] == dout.shape[1]) ||
                                  (bias.shape.rank == 2 && bias.shape[0] == 1 && bias.shape[1] == dout.shape[1]);
            if (!row_bias || producer.count(bias.id)) break;     // the bias must be a plain parameter or input
            if ((i < n_inference_nodes_) != (j < n_inference_nodes_) && n_inference_nodes_ != 0) break;
            lin_add_of_[i] = j;
            lin_dot_of_[j] = i;
            fwd_skip_[j] = 1;
            bwd_skip_[j] = 1;
            break;
        }
    }
    // nn.CrossEntropyLoss at the end of the graph: MAX, SUB, EXP, SUM, LOG, SUB (LogSoftmax along axis 1),
    // MUL by the targets, SUM, MUL by a literal -- nine nodes on [B, C] tensors, run as one call each way
    // when nothing else reads their intermediate results.
    for (int i = 0; i + 8 < nn; ++i) {
        auto N = [&](int k) -> const Node& { return g_.nodes[i + k]; };
        auto O = [&](int k) -> const Symbol& { return g_.nodes[i + k].outputs[0]; };
        static const int ops[9] = {MTL_OP_MAX, MTL_OP_SUB, MTL_OP_EXP, MTL_OP_SUM, MTL_OP_LOG, MTL_OP_SUB,
                                   MTL_OP_MUL, MTL_OP_SUM, MTL_OP_MUL};
        bool m = true;
        for (int k = 0; k < 9 && m; ++k) m = N(k).op == ops[k] && N(k).outputs.size() == 1;
        if (!m) continue;
        const Symbol& x = N(0).inputs[0];
        if (x.shape.rank != 2 || !x.trainable) continue;
        if (!N(0).attrs.axis || *N(0).attrs.axis != 1 || !N(3).attrs.axis || *N(3).attrs.axis != 1 || N(7).attrs.axis) continue;
        if (N(1).inputs.size() != 2 || N(5).inputs.size() != 2 || N(6).inputs.size() != 2 || N(8).inputs.size() != 2) continue;
        const Symbol& y = N(6).inputs[0];
        const Symbol& lit = N(8).inputs[1];
        m = N(1).inputs[0].id == x.id && N(1).inputs[1].id == O(0).id && N(2).inputs[0].id == O(1).id &&
            N(3).inputs[0].id == O(2).id && N(4).inputs[0].id == O(3).id && N(5).inputs[0].id == O(1).id &&
            N(5).inputs[1].id == O(4).id && N(6).inputs[1].id == O(5).id && N(7).inputs[0].id == O(6).id &&
            N(8).inputs[0].id == O(7).id && g_.loss_out && g_.loss_out->id == O(8).id;
        if (!m) continue;
        if (y.trainable || lit.trainable || !lit.shape.is_scalar() || !scalar_values_.count(lit.id)) continue;
        if (y.shape.rank != 2 || y.shape[0] != x.shape[0] || y.shape[1] != x.shape[1]) continue;
        if (x.shape.num_elements() > MTL_CROSS_ENTROPY_MAX_ELEMENTS) continue;
        if (n_inference_nodes_ > i) continue;   // part of the chain belongs to the inference graph
        static const int want_uses[8] = {1, 2, 1, 1, 1, 1, 1, 1};
        for (int k = 0; k < 8 && m; ++k) {
            m = uses[O(k).id] == want_uses[k] && !visible(O(k));
            for (auto& o : g_.outputs) if (o.id == O(k).id) m = false;
        }
        if (!m) continue;
        ce_head_ = i;
        ce_scale_sym_ = lit.id;
        ce_sole_reader_ = uses[x.id] == 2;   // MAX and the first SUB of this chain
        for (int k = 1; k < 9; ++k) { fwd_skip_[i + k] = 1; bwd_skip_[i + k] = 1; }
        break;
    }
}

static mtl_conv2d_desc conv_desc(const TensorShape& in, int K, int R, int S, const Attributes& a) {
    mtl_conv2d_desc d;
    d.N = (int32_t)in[0]; d.C = (int32_t)in[1]; d.H = (int32_t)in[2]; d.W = (int32_t)in[3];
    d.K = K; d.R = R; d.S = S;
    for (int i = 0; i < 2; ++i) { d.pad[i] = a.padding[i]; d.stride[i] = a.stride[i]; d.dilation[i] = a.dilation[i]; }
    return d;
}

static void unary_params(const Node& n, const std::map<int, float>& scalars, float* p0, float* p1) {
    *p0 = 0.0f;
    *p1 = 0.0f;
    if (n.op == MTL_OP_POW) {
        auto it = scalars.find(n.inputs[1].id);
        if (it == scalars.end()) throw Error(MTL_ERR_UNSUPPORTED, "POW exponent must be a graph scalar");
        *p0 = it->second;
    } else if (n.op == MTL_OP_LEAKYRELU) {
        *p0 = n.attrs.negative_slope;
    } else if (n.op == MTL_OP_CLIP) {
        *p0 = n.attrs.clip_min ? *n.attrs.clip_min : -3.402823466e38f;  // min_finite / max_finite
        *p1 = n.attrs.clip_max ? *n.attrs.clip_max : 3.402823466e38f;
    }
}

// A POW exponent that is trainable changes on the device with every optimizer step: read it back
// (4 bytes, waits for the stream) before it is used as a kernel argument.  Literal exponents -- every
// POW the reference's layers build -- keep the host copy taken at construction.
void Model::refresh_pow_exponent(const Node& n) {
    if (n.op != MTL_OP_POW || n.inputs.size() < 2 || !n.inputs[1].trainable) return;
    float v = 0.0f;
    check(mtl_d2h(ctx_, &v, T(n.inputs[1]), 4), "POW exponent read-back");
    scalar_values_[n.inputs[1].id] = v;
}

// forward_op, ops.mojo:243-352
void Model::forward_op(const Node& n) {
    const Symbol& out = n.outputs[0];
    const Symbol& t1 = n.inputs[0];
    float p0, p1;
    refresh_pow_exponent(n);
    switch (n.op) {
        case MTL_OP_CONCAT: {   // dynamics.mojo:25-108
            std::vector<const float*> ins;
            std::vector<int64_t> shapes;
            for (auto& s : n.inputs) {
                ins.push_back(T(s));
                shapes.insert(shapes.end(), s.shape.dims, s.shape.dims + s.shape.rank);
            }
            check(mtl_concat_fwd(ctx_, T(out), ins.data(), (int32_t)ins.size(), t1.shape.rank, shapes.data(), n.attrs.cat_dim),
                  "CONCAT forward");
            break;
        }
        case MTL_OP_SPLIT: {    // dynamics.mojo:111-199
            std::vector<float*> outs;
            for (auto& s : n.outputs) outs.push_back(T(s));
            check(mtl_split_fwd(ctx_, outs.data(), T(t1), (int32_t)outs.size(), t1.shape.rank, t1.shape.dims,
                                n.attrs.sections.data(), n.attrs.cat_dim), "SPLIT forward");
            break;
        }
        case MTL_OP_ADD: case MTL_OP_SUB: case MTL_OP_MUL: case MTL_OP_DIV:
            check(mtl_binary_fwd(ctx_, n.op, T(out), T(t1), T(n.inputs[1]), t1.shape.rank, t1.shape.dims,
                                 n.inputs[1].shape.rank, n.inputs[1].shape.dims), "binary forward");
            break;
        case MTL_OP_POW: case MTL_OP_EXP: case MTL_OP_LOG: case MTL_OP_SIGMOID: case MTL_OP_RELU:
        case MTL_OP_LEAKYRELU: case MTL_OP_TANH: case MTL_OP_CLIP:
            unary_params(n, scalar_values_, &p0, &p1);
            check(mtl_unary_fwd(ctx_, n.op, T(out), T(t1), t1.shape.num_elements(), p0, p1), "unary forward");
            break;
        case MTL_OP_DOT: {
            const int self = (int)(&n - &g_.nodes[0]);
            if (fusion_ && lin_add_of_[self] >= 0) {
                const Node& add = g_.nodes[lin_add_of_[self]];
                check(mtl_linear_fwd(ctx_, T(add.outputs[0]), T(t1), T(n.inputs[1]), T(add.inputs[1]), t1.shape[0], t1.shape[1],
                                     n.inputs[1].shape[1]), "Linear forward");
                break;
            }
            check(mtl_dot_fwd(ctx_, T(out), T(t1), T(n.inputs[1]), t1.shape[0], t1.shape[1], n.inputs[1].shape[1]),
                  "DOT forward");
            break;
        }
        case MTL_OP_SUM: case MTL_OP_MEAN: case MTL_OP_MAX:
            check(mtl_reduce_fwd(ctx_, n.op, T(out), T(t1), t1.shape.rank, t1.shape.dims,
                                 n.attrs.axis ? *n.attrs.axis : -1), "reduce forward");
            break;
        case MTL_OP_FLATTEN: case MTL_OP_RESHAPE: case MTL_OP_SQUEEZE: case MTL_OP_UNSQUEEZE:
            if (alias_node_[(size_t)(&n - &g_.nodes[0])]) break;   // the result shares its operand's storage
            check(mtl_copy_f32(ctx_, T(out), T(t1), t1.shape.num_elements(), 0), "copy forward");
            break;
        case MTL_OP_CONV2D: {
            const Symbol& w = n.inputs[1];
            mtl_conv2d_desc d = conv_desc(t1.shape, (int)w.shape[0], (int)w.shape[2], (int)w.shape[3], n.attrs);
            const int self = (int)(&n - &g_.nodes[0]);
            if (fusion_ && fwd_pool_of_[self] >= 0) {
                const int pk = fwd_pool_of_[self];
                const Node& q = g_.nodes[pk];
                mtl_conv2d_desc pd = conv_desc(q.inputs[0].shape, 1, q.attrs.kernel_size[0], q.attrs.kernel_size[1], q.attrs);
                float* out_cl = twins_.count(q.outputs[0].id) ? twins_.at(q.outputs[0].id) : nullptr;
                check(mtl_conv2d_fwd_act_pool_cl(ctx_, T(q.outputs[0]), pool_idx_.at(pk), out_cl, T(t1), twin_of(t1), T(w),
                                                 T(n.inputs[2]), &d, MTL_OP_RELU, &pd), "CONV2D+RELU+MAXPOOL2D forward");
                if (out_cl) twin_valid_[q.outputs[0].id] = true;
            } else if (fusion_ && fwd_relu_of_[self] >= 0)
                check(mtl_conv2d_fwd_act(ctx_, T(g_.nodes[fwd_relu_of_[self]].outputs[0]), T(t1), T(w), T(n.inputs[2]), &d,
                                         MTL_OP_RELU), "CONV2D+RELU forward");
            else
                check(mtl_conv2d_fwd(ctx_, T(out), T(t1), T(w), T(n.inputs[2]), &d), "CONV2D forward");
            break;
        }
        case MTL_OP_MAXPOOL2D: {
            mtl_conv2d_desc d = conv_desc(t1.shape, 1, n.attrs.kernel_size[0], n.attrs.kernel_size[1], n.attrs);
            int node_index = (int)(&n - &g_.nodes[0]);
            check(mtl_maxpool2d_fwd(ctx_, T(out), pool_idx_.at(node_index), T(t1), &d), "MAXPOOL2D forward");
            break;
        }
        case MTL_OP_FMA:
            check(mtl_fma_fwd(ctx_, T(out), T(t1), T(n.inputs[1]), T(n.inputs[2]), t1.shape.num_elements()), "FMA forward");
            break;
        case MTL_OP_TRANSPOSE:
            check(mtl_transpose_fwd(ctx_, T(out), T(t1), t1.shape.rank, t1.shape.dims,
                                    n.attrs.axes.empty() ? nullptr : n.attrs.axes.data()), "TRANSPOSE forward");
            break;
        case MTL_OP_SLICE: {
            mtl_slice_desc d = Graph::slice_desc(n.attrs);
            check(mtl_slice_fwd(ctx_, T(out), T(t1), t1.shape.rank, t1.shape.dims, &d), "SLICE forward");
            break;
        }
        default:
            throw Error(MTL_ERR_UNSUPPORTED, "operator id " + std::to_string(n.op) + " is not on the GPU path");
    }
}

int Model::acc_flag(const Symbol& s) {
    if (!overwrite_first_) return 1;
    bool& w = grad_written_[s.id];
    if (w) return 1;
    w = true;
    return 0;
}

// backward_op, ops.mojo:355-528: grad(operand tensor_id) += local gradient
void Model::backward_op(const Node& n, int tensor_id) {
    const Symbol& out = n.outputs[0];
    const Symbol& t1 = n.inputs[0];
    const Symbol& tj = n.inputs[tensor_id];
    float* ug = G(out);
    float* grad = G(tj);
    int acc = acc_flag(tj);
    float p0, p1;
    refresh_pow_exponent(n);
    switch (n.op) {
        case MTL_OP_CONCAT: {
            std::vector<int64_t> shapes;
            for (auto& s : n.inputs) shapes.insert(shapes.end(), s.shape.dims, s.shape.dims + s.shape.rank);
            check(mtl_concat_bwd(ctx_, grad, ug, tensor_id, (int32_t)n.inputs.size(), t1.shape.rank, shapes.data(),
                                 n.attrs.cat_dim, acc), "CONCAT backward");
            break;
        }
        case MTL_OP_SPLIT: {   // the operand's gradient gathers the gradients of all the pieces
            std::vector<const float*> ugs;
            for (auto& s : n.outputs) ugs.push_back(G(s));
            check(mtl_split_bwd(ctx_, grad, ugs.data(), (int32_t)ugs.size(), t1.shape.rank, t1.shape.dims,
                                n.attrs.sections.data(), n.attrs.cat_dim, acc), "SPLIT backward");
            break;
        }
        case MTL_OP_ADD: case MTL_OP_SUB: case MTL_OP_MUL: case MTL_OP_DIV:
            check(mtl_binary_bwd(ctx_, n.op, tensor_id, grad, ug, T(t1), T(n.inputs[1]), t1.shape.rank, t1.shape.dims,
                                 n.inputs[1].shape.rank, n.inputs[1].shape.dims, acc), "binary backward");
            break;
        case MTL_OP_POW:
            if (tensor_id == 1) {   // basics.mojo:359-376: the exponent's gradient is a sum over all elements
                unary_params(n, scalar_values_, &p0, &p1);
                check(mtl_pow_bwd_exponent(ctx_, grad, ug, T(t1), t1.shape.num_elements(), p0, acc), "POW exponent backward");
                break;
            }
            // fallthrough
        case MTL_OP_EXP: case MTL_OP_LOG: case MTL_OP_SIGMOID: case MTL_OP_RELU: case MTL_OP_LEAKYRELU:
        case MTL_OP_TANH: case MTL_OP_CLIP:
            unary_params(n, scalar_values_, &p0, &p1);
            // a RELU whose input was never written (fused into its CONV2D): out > 0 exactly where in > 0
            check(mtl_unary_bwd(ctx_, n.op, grad, ug,
                                (fusion_ && n.op == MTL_OP_RELU && relu_in_absent_[(int)(&n - &g_.nodes[0])]) ? T(out) : T(t1),
                                t1.shape.num_elements(), p0, p1, acc), "unary backward");
            break;
        case MTL_OP_DOT:
            check(mtl_dot_bwd(ctx_, tensor_id, grad, ug, T(t1), T(n.inputs[1]), t1.shape[0], t1.shape[1],
                              n.inputs[1].shape[1], acc), "DOT backward");
            break;
        case MTL_OP_SUM: case MTL_OP_MEAN: case MTL_OP_MAX:
            check(mtl_reduce_bwd(ctx_, n.op, grad, ug, T(t1), t1.shape.rank, t1.shape.dims,
                                 n.attrs.axis ? *n.attrs.axis : -1, acc), "reduce backward");
            break;
        case MTL_OP_FLATTEN: case MTL_OP_RESHAPE: case MTL_OP_SQUEEZE: case MTL_OP_UNSQUEEZE:
            // shared storage: the operand's gradient IS the result's gradient (this node is its only writer)
            if (alias_node_[(size_t)(&n - &g_.nodes[0])]) break;
            check(mtl_copy_f32(ctx_, grad, ug, t1.shape.num_elements(), acc), "copy backward");
            break;
        case MTL_OP_CONV2D: {
            const Symbol& w = n.inputs[1];
            mtl_conv2d_desc d = conv_desc(t1.shape, (int)w.shape[0], (int)w.shape[2], (int)w.shape[3], n.attrs);
            check(mtl_conv2d_bwd(ctx_, tensor_id, grad, ug, T(t1), T(w), &d, acc), "CONV2D backward");
            break;
        }
        case MTL_OP_MAXPOOL2D: {
            mtl_conv2d_desc d = conv_desc(t1.shape, 1, n.attrs.kernel_size[0], n.attrs.kernel_size[1], n.attrs);
            int node_index = (int)(&n - &g_.nodes[0]);
            // the indices stored by this step's forward pass select the same elements the
            // reference finds by re-scanning the input (pool.mojo:123-163)
            if (fusion_ && bwd_relu_of_[node_index] >= 0) {
                // acc was taken for the RELU output's gradient, which is not written: release it
                grad_written_[tj.id] = false;
                const Symbol& rin = g_.nodes[bwd_relu_of_[node_index]].inputs[0];
                check(mtl_maxpool2d_bwd_idx_act(ctx_, G(rin), ug, pool_idx_.at(node_index), T(out), &d, MTL_OP_RELU,
                                                acc_flag(rin)), "MAXPOOL2D+RELU backward");
            } else {
                check(mtl_maxpool2d_bwd_idx(ctx_, grad, ug, pool_idx_.at(node_index), &d, acc), "MAXPOOL2D backward");
            }
            break;
        }
        case MTL_OP_FMA:
            check(mtl_fma_bwd(ctx_, tensor_id, grad, ug, T(t1), T(n.inputs[1]), t1.shape.num_elements(), acc), "FMA backward");
            break;
        case MTL_OP_TRANSPOSE:
            check(mtl_transpose_bwd(ctx_, grad, ug, t1.shape.rank, t1.shape.dims,
                                    n.attrs.axes.empty() ? nullptr : n.attrs.axes.data(), acc), "TRANSPOSE backward");
            break;
        case MTL_OP_SLICE: {
            mtl_slice_desc d = Graph::slice_desc(n.attrs);
            check(mtl_slice_bwd(ctx_, grad, ug, t1.shape.rank, t1.shape.dims, &d, acc), "SLICE backward");
            break;
        }
        default:
            throw Error(MTL_ERR_UNSUPPORTED, "operator id " + std::to_string(n.op) + " is not on the GPU path");
    }
}

void Model::backward_enqueue() {
    if (!g_.loss_out) throw Error(MTL_ERR_INVALID, "no loss defined");
    if (profiling_) ++bwd_passes_;
    grad_written_.clear();
    // fill(grads[loss], 1.0), model.mojo:180
    // (not needed when the loss chain runs as mtl_cross_entropy_bwd, which assumes the seed)
    if (!(fusion_ && ce_head_ >= 0))
        check(mtl_fill_f32(ctx_, G(*g_.loss_out), g_.loss_out->shape.num_elements(), 1.0f), "seed loss gradient");
    grad_written_[g_.loss_out->id] = true;
    // While a fused CONV2D backward runs, the library reports the moment its parameter gradients are
    // enqueued (before the input gradient's kernels): the node's after_backward_node call is made
    // then, so that a data-parallel trainer's exchange of those gradients overlaps the rest of the node.
    struct EarlyHook {
        Model* m; int node; bool fired = false; bool armed;
        EarlyHook(Model* m_, int node_, bool arm) : m(m_), node(node_), armed(arm && m_->after_backward_node) {
            if (armed) mtl_set_grads_ready_hook(m->ctx_, &EarlyHook::call, this);
        }
        ~EarlyHook() { if (armed) mtl_set_grads_ready_hook(m->ctx_, nullptr, nullptr); }
        std::exception_ptr error;   // an exception must not travel through the C frames of the library
        static void call(void* self) {
            EarlyHook* h = static_cast<EarlyHook*>(self);
            if (h->fired) return;
            h->fired = true;
            try { h->m->after_backward_node(h->m->after_backward_user, h->node); }
            catch (...) { h->error = std::current_exception(); }
        }
        void rethrow() { if (error) std::rethrow_exception(error); }
    };
    for (int i = (int)g_.nodes.size() - 1; i >= 0; --i) {
        const Node& n = g_.nodes[i];
        bool node_reported = false;
        NodeRange range(ctx_, profiling_ && !(fusion_ && (bwd_skip_[i] || bwd_pool_skip_[i])), kBackwardTag + i);
        if (fusion_ && (bwd_skip_[i] || bwd_pool_skip_[i])) {
            // a RELU whose backward its MAXPOOL2D performs, or a MAXPOOL2D whose backward the CONV2D at
            // the head of the chain performs from the pooled gradient
        } else if (fusion_ && i == ce_head_) {
            // the nine backward calls of the loss chain, gradient seed 1 included
            const Symbol& x = n.inputs[0];
            const int acc = acc_flag(x);
            if (ce_grad_fresh_ && !acc) {
                ce_grad_fresh_ = false;   // written by the forward launch; a second backward pass recomputes it
            } else {
                check(mtl_cross_entropy_bwd(ctx_, G(x), T(x), T(g_.nodes[i + 6].inputs[0]), x.shape[0], x.shape[1],
                                            scalar_values_.at(ce_scale_sym_), acc), "CrossEntropyLoss backward");
            }
        } else if (fusion_ && n.op == MTL_OP_DOT && lin_add_of_[i] >= 0) {
            // DOT.backward for both operands and the bias ADD's backward, from the gradient of the ADD's result
            const Node& add = g_.nodes[lin_add_of_[i]];
            const Symbol& a = n.inputs[0];
            const Symbol& w = n.inputs[1];
            const Symbol& b = add.inputs[1];
            float* da = a.trainable ? G(a) : nullptr;
            float* dw = w.trainable ? G(w) : nullptr;
            float* db = b.trainable ? G(b) : nullptr;
            const int xa = da ? acc_flag(a) : 0, xw = dw ? acc_flag(w) : 0, xb = db ? acc_flag(b) : 0;
            check(mtl_linear_bwd(ctx_, da, dw, db, G(add.outputs[0]), T(a), T(w), a.shape[0], a.shape[1], w.shape[1], xa, xw, xb),
                  "Linear backward");
        } else if (fusion_ && n.op == MTL_OP_CONV2D && bwd_pooled_of_[i] >= 0) {
            const Node& q = g_.nodes[bwd_pooled_of_[i]];  // the MAXPOOL2D at the end of the chain
            const Symbol& x = n.inputs[0];
            const Symbol& w = n.inputs[1];
            const Symbol& b = n.inputs[2];
            mtl_conv2d_desc d = conv_desc(x.shape, (int)w.shape[0], (int)w.shape[2], (int)w.shape[3], n.attrs);
            mtl_conv2d_desc pd = conv_desc(q.inputs[0].shape, 1, q.attrs.kernel_size[0], q.attrs.kernel_size[1], q.attrs);
            float* dx = x.trainable ? G(x) : nullptr;
            float* dw = w.trainable ? G(w) : nullptr;
            float* db = b.trainable ? G(b) : nullptr;
            const int ax = dx ? acc_flag(x) : 0, aw = dw ? acc_flag(w) : 0, ab = db ? acc_flag(b) : 0;
            if (dx || dw || db) {
                EarlyHook early(this, i, dx != nullptr);
                check(mtl_conv2d_bwd_pooled(ctx_, dx, dw, db, G(q.outputs[0]), pool_idx_.at(bwd_pooled_of_[i]), T(q.outputs[0]),
                                            T(x), twin_of(x), T(w), &d, MTL_OP_RELU, &pd, ax, aw, ab),
                      "CONV2D backward from the pooled gradient");
                early.rethrow();
                node_reported = early.fired;
            }
        } else if (fusion_ && n.op == MTL_OP_CONV2D) {
            // all wanted operand gradients of the layer from one pass over ug (mtl_conv2d_bwd_fused)
            const Symbol& x = n.inputs[0];
            const Symbol& w = n.inputs[1];
            const Symbol& b = n.inputs[2];
            mtl_conv2d_desc d = conv_desc(x.shape, (int)w.shape[0], (int)w.shape[2], (int)w.shape[3], n.attrs);
            float* dx = x.trainable ? G(x) : nullptr;
            float* dw = w.trainable ? G(w) : nullptr;
            float* db = b.trainable ? G(b) : nullptr;
            const int ax = dx ? acc_flag(x) : 0, aw = dw ? acc_flag(w) : 0, ab = db ? acc_flag(b) : 0;
            if (dx || dw || db) {
                EarlyHook early(this, i, dx != nullptr);
                check(mtl_conv2d_bwd_fused_cl(ctx_, dx, dw, db, G(n.outputs[0]), T(x), twin_of(x), T(w), &d, ax, aw, ab),
                      "CONV2D backward");
                early.rethrow();
                node_reported = early.fired;
            }
        } else {
            for (int j = 0; j < (int)n.inputs.size(); ++j)
                if (n.inputs[j].trainable) backward_op(n, j);
        }
        if (after_backward_node && !node_reported) after_backward_node(after_backward_user, i);
    }
}

void Model::backward() { backward_enqueue(); }

// ------------------------------------------------------------------ Adam -------------------

Adam::Adam(Model& model, float lr, float beta1, float beta2, float epsilon)
    : model_(model), lr_(lr), beta1_(beta1), beta2_(beta2), eps_(epsilon) {
    mtl_ctx* ctx = model_.ctx();
    size_t bytes = (size_t)std::max<int64_t>(model_.n_trainable(), 1) * 4;
    auto ck = [&](int rc, const char* w) {
        if (rc != MTL_OK) throw Error(rc, std::string(w) + ": " + mtl_last_error(ctx));
    };
    // allocate_rms_and_momentum (optim.mojo:142-149): zero-initialised
    ck(mtl_malloc(ctx, bytes, (void**)&m_), "Adam momentum");
    ck(mtl_malloc(ctx, bytes, (void**)&v_), "Adam rms");
    ck(mtl_malloc(ctx, 4, (void**)&t_dev_), "Adam counter");
    ck(mtl_zero(ctx, m_, bytes), "zero momentum");
    ck(mtl_zero(ctx, v_, bytes), "zero rms");
    ck(mtl_zero(ctx, t_dev_, 4), "zero counter");
}

Adam::~Adam() {
    mtl_free(model_.ctx(), m_);
    mtl_free(model_.ctx(), v_);
    mtl_free(model_.ctx(), t_dev_);
}

// Both forms advance the SAME counter: the one in device memory is what the update reads (so that a
// captured step can be replayed), iter_ is its host copy.  Eager steps and Trainer steps may
// therefore be mixed on one optimizer without the bias corrections 1 - beta^t going stale.
void Adam::step() { step_captured(); }  // optim.mojo:94-140

void Adam::step_captured() {
    iter_ += 1;  // optim.mojo:96
    int rc = mtl_adam_step_dev(model_.ctx(), model_.params_flat(), model_.grads_flat(), m_, v_, model_.n_trainable(),
                               lr_, beta1_, beta2_, eps_, t_dev_, grad_scale_);
    if (rc != MTL_OK) throw Error(rc, std::string("Adam.step: ") + mtl_last_error(model_.ctx()));
}

void Adam::set_state(int which, const float* host_in) {
    int rc = mtl_h2d(model_.ctx(), which == 0 ? m_ : v_, host_in, (size_t)model_.n_trainable() * 4);
    if (rc != MTL_OK) throw Error(rc, std::string("Adam state upload: ") + mtl_last_error(model_.ctx()));
}

void Adam::set_iter(int iter) {
    iter_ = iter;
    int32_t t = iter;
    int rc = mtl_h2d(model_.ctx(), t_dev_, &t, 4);
    if (rc != MTL_OK) throw Error(rc, std::string("Adam counter upload: ") + mtl_last_error(model_.ctx()));
}

void Adam::get_state(int which, float* host_out) const {
    int rc = mtl_d2h(model_.ctx(), host_out, which == 0 ? m_ : v_, (size_t)model_.n_trainable() * 4);
    if (rc != MTL_OK) throw Error(rc, std::string("Adam state read-back: ") + mtl_last_error(model_.ctx()));
}

}  // namespace mantle
