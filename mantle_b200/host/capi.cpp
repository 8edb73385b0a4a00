// Flat C interface to the host mirror (Graph / Model / Adam / Trainer and the nn builders) so
// that tests and the benchmark can drive it through ctypes.  Every function returns an mtl_status
// code; the message of the last failure on the calling thread is at mtlh_last_error().
#include <cstring>
#include <map>
#include <string>

#include "nn.hpp"
#include "checkpoint.hpp"
#include "trainer.hpp"

#define MTLH_API extern "C" __attribute__((visibility("default")))

using namespace mantle;

namespace {

thread_local std::string g_err;

struct GraphBox {
    Graph g;
    std::map<int, Symbol> syms;
    void remember(const Symbol& s) { syms[s.id] = s; }
    void rescan() {
        for (auto& s : g.inputs) remember(s);
        for (auto& s : g.params) remember(s);
        for (auto& n : g.nodes)
            for (auto& s : n.outputs) remember(s);
    }
    const Symbol& sym(int id) const {
        auto it = syms.find(id);
        if (it == syms.end()) throw Error(MTL_ERR_INVALID, "unknown symbol id " + std::to_string(id));
        return it->second;
    }
};

template <class F>
int guard(F&& f) {
    try {
        f();
        return MTL_OK;
    } catch (const Error& e) {
        g_err = e.what();
        return e.code;
    } catch (const std::exception& e) {
        g_err = e.what();
        return MTL_ERR_INVALID;
    }
}

}  // namespace

// Attribute block passed from the binding; has_* flags mark the optional entries.
struct mtlh_attrs {
    int32_t has_axis, axis;
    int32_t shape_rank;
    int64_t shape[MTL_MAX_RANK];
    int32_t padding[2], stride[2], dilation[2], kernel_size[2];
    float negative_slope;
    int32_t has_clip_min, has_clip_max;
    float clip_min, clip_max;
    int32_t n_dims;
    int32_t dims[MTL_MAX_RANK];
    int32_t n_axes;
    int32_t axes[MTL_MAX_RANK];
    int32_t n_slice, has_steps;
    int64_t starts[MTL_MAX_RANK], ends[MTL_MAX_RANK], steps[MTL_MAX_RANK];
};

static Attributes to_attrs(const mtlh_attrs* a) {
    Attributes r;
    if (!a) return r;
    if (a->has_axis) r.axis = a->axis;
    if (a->shape_rank > 0) r.shape = TensorShape(a->shape_rank, a->shape);
    for (int i = 0; i < 2; ++i) {
        r.padding[i] = a->padding[i];
        r.stride[i] = a->stride[i] > 0 ? a->stride[i] : 1;
        r.dilation[i] = a->dilation[i] > 0 ? a->dilation[i] : 1;
        r.kernel_size[i] = a->kernel_size[i];
    }
    r.negative_slope = a->negative_slope;
    if (a->has_clip_min) r.clip_min = a->clip_min;
    if (a->has_clip_max) r.clip_max = a->clip_max;
    for (int i = 0; i < a->n_dims && i < MTL_MAX_RANK; ++i) r.dims.push_back(a->dims[i]);
    for (int i = 0; i < a->n_axes && i < MTL_MAX_RANK; ++i) r.axes.push_back(a->axes[i]);
    for (int i = 0; i < a->n_slice && i < MTL_MAX_RANK; ++i) {
        r.starts.push_back(a->starts[i]);
        r.ends.push_back(a->ends[i]);
        if (a->has_steps) r.steps.push_back(a->steps[i]);
    }
    return r;
}

MTLH_API const char* mtlh_last_error(void) { return g_err.c_str(); }

// ------------------------------------------------------------------ Graph -----------------

MTLH_API int32_t mtlh_graph_create(void** out) {
    return guard([&] { *out = new GraphBox(); });
}
MTLH_API int32_t mtlh_graph_destroy(void* g) {
    delete static_cast<GraphBox*>(g);
    return MTL_OK;
}
MTLH_API int32_t mtlh_graph_input(void* g, int32_t rank, const int64_t* shape, int32_t trainable, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        Symbol s = b->g.input(TensorShape(rank, shape), trainable != 0);
        b->remember(s);
        *out_id = s.id;
    });
}
// kind: 0 zero, 1 data, 2 uniform(lo, hi)
MTLH_API int32_t mtlh_graph_param(void* g, int32_t rank, const int64_t* shape, int32_t kind, const float* data,
                                  int64_t n_data, float lo, float hi, int32_t trainable, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        Param p;
        p.kind = kind == 1 ? Param::DATA : kind == 2 ? Param::UNIFORM : Param::ZERO;
        if (kind == 1 && data) p.data.assign(data, data + n_data);
        p.lo = lo;
        p.hi = hi;
        Symbol s = b->g.param(TensorShape(rank, shape), p, trainable != 0);
        b->remember(s);
        *out_id = s.id;
    });
}
MTLH_API int32_t mtlh_graph_scalar(void* g, float value, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        Symbol s = b->g.scalar(value);
        b->remember(s);
        *out_id = s.id;
    });
}
MTLH_API int32_t mtlh_graph_op(void* g, int32_t op, int32_t n_operands, const int32_t* operand_ids,
                               const mtlh_attrs* attrs, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        std::vector<Symbol> ops;
        for (int i = 0; i < n_operands; ++i) ops.push_back(b->sym(operand_ids[i]));
        Symbol s = b->g.op(op, ops, to_attrs(attrs));
        b->remember(s);
        *out_id = s.id;
    });
}
// g.concat(*operands, dim) and g.split(operand, sections, dim): graph.mojo:180-210
MTLH_API int32_t mtlh_graph_concat(void* g, int32_t n_operands, const int32_t* operand_ids, int32_t dim, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        std::vector<Symbol> ops;
        for (int i = 0; i < n_operands; ++i) ops.push_back(b->sym(operand_ids[i]));
        Symbol s = b->g.concat(ops, dim);
        b->remember(s);
        *out_id = s.id;
    });
}
MTLH_API int32_t mtlh_graph_split(void* g, int32_t operand_id, int32_t n_sections, const int64_t* sections, int32_t dim,
                                  int32_t* out_ids) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        std::vector<int64_t> sec(sections, sections + n_sections);
        std::vector<Symbol> res = b->g.split(b->sym(operand_id), sec, dim);
        for (size_t i = 0; i < res.size(); ++i) {
            b->remember(res[i]);
            out_ids[i] = res[i].id;
        }
    });
}
// g.op(op, symbol, literal) / g.op(op, literal, symbol): graph.mojo:131-157
MTLH_API int32_t mtlh_graph_op_scalar(void* g, int32_t op, int32_t sym_id, double value, int32_t scalar_first,
                                      const mtlh_attrs* attrs, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        Symbol s = scalar_first ? b->g.op(op, value, b->sym(sym_id), to_attrs(attrs))
                                : b->g.op(op, b->sym(sym_id), value, to_attrs(attrs));
        b->rescan();
        *out_id = s.id;
    });
}
MTLH_API int32_t mtlh_graph_out(void* g, int32_t id) {
    return guard([&] { auto* b = static_cast<GraphBox*>(g); b->g.out(b->sym(id)); });
}
MTLH_API int32_t mtlh_graph_loss(void* g, int32_t id) {
    return guard([&] { auto* b = static_cast<GraphBox*>(g); b->g.loss(b->sym(id)); });
}
MTLH_API int32_t mtlh_graph_symbol(void* g, int32_t id, int32_t* rank, int64_t* dims, int32_t* trainable) {
    return guard([&] {
        const Symbol& s = static_cast<GraphBox*>(g)->sym(id);
        *rank = s.shape.rank;
        for (int i = 0; i < s.shape.rank; ++i) dims[i] = s.shape.dims[i];
        *trainable = s.trainable;
    });
}
MTLH_API int32_t mtlh_graph_counts(void* g, int32_t* n_nodes, int32_t* n_params, int32_t* n_inputs, int32_t* n_symbols) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        *n_nodes = (int)b->g.nodes.size();
        *n_params = (int)b->g.params.size();
        *n_inputs = (int)b->g.inputs.size();
        *n_symbols = b->g.symbol_count;
    });
}
MTLH_API int32_t mtlh_graph_node(void* g, int32_t i, int32_t* op, int32_t* n_in, int32_t* in_ids, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        if (i < 0 || i >= (int)b->g.nodes.size()) throw Error(MTL_ERR_INVALID, "node index out of range");
        const Node& n = b->g.nodes[i];
        *op = n.op;
        *n_in = (int)n.inputs.size();
        for (size_t j = 0; j < n.inputs.size() && j < 8; ++j) in_ids[j] = n.inputs[j].id;
        *out_id = n.outputs[0].id;
    });
}
MTLH_API int32_t mtlh_graph_param_id(void* g, int32_t i, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        if (i < 0 || i >= (int)b->g.params.size()) throw Error(MTL_ERR_INVALID, "parameter index out of range");
        *out_id = b->g.params[i].id;
    });
}

// ------------------------------------------------------------------ nn builders -----------

MTLH_API int32_t mtlh_nn_linear(void* g, int32_t x, int32_t n_outputs, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        Symbol s = nn::Linear(b->g, b->sym(x), n_outputs);
        b->rescan();
        *out_id = s.id;
    });
}
MTLH_API int32_t mtlh_nn_conv2d(void* g, int32_t x, int32_t out_channels, const int32_t* k, const int32_t* pad,
                                const int32_t* stride, const int32_t* dil, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        Symbol s = nn::Conv2d(b->g, b->sym(x), out_channels, k[0], k[1], pad[0], pad[1], stride[0], stride[1], dil[0], dil[1]);
        b->rescan();
        *out_id = s.id;
    });
}
MTLH_API int32_t mtlh_nn_maxpool2d(void* g, int32_t x, const int32_t* k, const int32_t* stride, const int32_t* pad,
                                   const int32_t* dil, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        Symbol s = nn::MaxPool2d(b->g, b->sym(x), k[0], k[1], stride[0], stride[1], pad[0], pad[1], dil[0], dil[1]);
        b->rescan();
        *out_id = s.id;
    });
}
// which: 0 Softmax, 1 LogSoftmax
MTLH_API int32_t mtlh_nn_softmax(void* g, int32_t x, int32_t axis, int32_t which, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        Symbol s = which ? nn::LogSoftmax(b->g, b->sym(x), axis) : nn::Softmax(b->g, b->sym(x), axis);
        b->rescan();
        *out_id = s.id;
    });
}
// which: 0 MSELoss, 1 CrossEntropyLoss
MTLH_API int32_t mtlh_nn_loss(void* g, int32_t y_pred, int32_t y_true, int32_t which, int32_t* out_id) {
    return guard([&] {
        auto* b = static_cast<GraphBox*>(g);
        Symbol s = which ? nn::CrossEntropyLoss(b->g, b->sym(y_pred), b->sym(y_true))
                         : nn::MSELoss(b->g, b->sym(y_pred), b->sym(y_true));
        b->rescan();
        *out_id = s.id;
    });
}

// ------------------------------------------------------------------ Model -----------------

MTLH_API int32_t mtlh_model_create(mtl_ctx* ctx, void* g, uint64_t seed, void** out) {
    return guard([&] { *out = new Model(ctx, static_cast<GraphBox*>(g)->g, seed); });
}
MTLH_API int32_t mtlh_model_destroy(void* m) {
    delete static_cast<Model*>(m);
    return MTL_OK;
}
MTLH_API int32_t mtlh_model_forward(void* m, int32_t n_in, const float* const* inputs, float* loss) {
    return guard([&] {
        std::vector<const float*> in(inputs, inputs + n_in);
        *loss = static_cast<Model*>(m)->forward(in);
    });
}
MTLH_API int32_t mtlh_model_inference(void* m, int32_t n_in, const float* const* inputs, int32_t n_out,
                                      float* const* outputs) {
    return guard([&] {
        std::vector<const float*> in(inputs, inputs + n_in);
        std::vector<float*> out(outputs, outputs + n_out);
        static_cast<Model*>(m)->inference(in, out);
    });
}
MTLH_API int32_t mtlh_model_backward(void* m) {
    return guard([&] { static_cast<Model*>(m)->backward(); });
}
MTLH_API int32_t mtlh_model_zero_grads(void* m) {
    return guard([&] { static_cast<Model*>(m)->zero_grads(); });
}
MTLH_API int32_t mtlh_model_get_tensor(void* m, int32_t id, float* host_out) {
    return guard([&] { static_cast<Model*>(m)->get_tensor(id, host_out); });
}
MTLH_API int32_t mtlh_model_set_tensor(void* m, int32_t id, const float* host_in) {
    return guard([&] { static_cast<Model*>(m)->set_tensor(id, host_in); });
}
MTLH_API int32_t mtlh_model_get_grad(void* m, int32_t id, float* host_out) {
    return guard([&] { static_cast<Model*>(m)->get_grad(id, host_out); });
}
MTLH_API int32_t mtlh_model_set_overwrite_first(void* m, int32_t on) {
    return guard([&] { static_cast<Model*>(m)->set_overwrite_first(on != 0); });
}
MTLH_API int32_t mtlh_model_set_fusion(void* m, int32_t on) {
    return guard([&] { static_cast<Model*>(m)->set_fusion(on != 0); });
}
MTLH_API int64_t mtlh_model_n_trainable(void* m) { return static_cast<Model*>(m)->n_trainable(); }
MTLH_API int32_t mtlh_model_n_inference_nodes(void* m) { return static_cast<Model*>(m)->n_inference_nodes(); }
// Symbol ids and flat offsets of the trainable parameters, in optimizer order.
MTLH_API int32_t mtlh_model_trainable(void* m, int32_t cap, int32_t* ids, int64_t* offsets, int32_t* n) {
    return guard([&] {
        auto* mm = static_cast<Model*>(m);
        *n = (int)mm->trainable_parameters().size();
        for (int i = 0; i < *n && i < cap; ++i) {
            ids[i] = mm->trainable_parameters()[i].id;
            offsets[i] = mm->trainable_offsets()[i];
        }
    });
}

// ------------------------------------------------------------------ Adam ------------------

MTLH_API int32_t mtlh_adam_create(void* m, float lr, float beta1, float beta2, float eps, void** out) {
    return guard([&] { *out = new Adam(*static_cast<Model*>(m), lr, beta1, beta2, eps); });
}
MTLH_API int32_t mtlh_adam_destroy(void* a) {
    delete static_cast<Adam*>(a);
    return MTL_OK;
}
MTLH_API int32_t mtlh_adam_zero_grad(void* a) {
    return guard([&] { static_cast<Adam*>(a)->zero_grad(); });
}
MTLH_API int32_t mtlh_adam_step(void* a) {
    return guard([&] { static_cast<Adam*>(a)->step(); });
}
MTLH_API int32_t mtlh_adam_iter(void* a) { return static_cast<Adam*>(a)->iter(); }
MTLH_API int32_t mtlh_adam_get_state(void* a, int32_t which, float* host_out) {
    return guard([&] { static_cast<Adam*>(a)->get_state(which, host_out); });
}

MTLH_API int32_t mtlh_adam_set_state(void* a, int32_t which, const float* host_in) {
    return guard([&] { static_cast<Adam*>(a)->set_state(which, host_in); });
}
MTLH_API int32_t mtlh_adam_set_iter(void* a, int32_t iter) {
    return guard([&] { static_cast<Adam*>(a)->set_iter(iter); });
}
// Offsets (in floats) of the trainable parameters inside the flat spans, in get_trainable_parameters order.
MTLH_API int32_t mtlh_model_trainable_offsets(void* m, int64_t* out, int32_t cap, int32_t* n) {
    return guard([&] {
        const auto& off = static_cast<Model*>(m)->trainable_offsets();
        for (size_t i = 0; i < off.size() && (int32_t)i < cap; ++i) out[i] = off[i];
        if (n) *n = (int32_t)off.size();
    });
}

// PerfMetrics (perf_utils.mojo:60-236): per-node device time
MTLH_API int32_t mtlh_model_set_profiling(void* m, int32_t on) {
    return guard([&] { static_cast<Model*>(m)->set_profiling(on != 0); });
}
// per node i: out[4 * i + 0..3] = forward ms, backward ms, forward launches, backward launches (sums over the passes)
MTLH_API int32_t mtlh_model_perf_metrics(void* m, double* out, int32_t n_nodes, int32_t* fwd_passes, int32_t* bwd_passes) {
    return guard([&] {
        int fp = 0, bp = 0;
        auto v = static_cast<Model*>(m)->perf_metrics(&fp, &bp);
        for (size_t i = 0; i < v.size() && (int32_t)i < n_nodes; ++i) {
            out[4 * i] = v[i].fwd_ms; out[4 * i + 1] = v[i].bwd_ms;
            out[4 * i + 2] = (double)v[i].fwd_launches; out[4 * i + 3] = (double)v[i].bwd_launches;
        }
        if (fwd_passes) *fwd_passes = fp;
        if (bwd_passes) *bwd_passes = bp;
    });
}
// print_forward_perf_metrics / print_backward_perf_metrics: the table as text (truncated to cap - 1 bytes)
MTLH_API int32_t mtlh_model_perf_report(void* m, int32_t forward, const char* time_format, int32_t print_shape, char* buf,
                                        int64_t cap) {
    return guard([&] {
        std::string r = static_cast<Model*>(m)->perf_report(forward != 0, time_format ? time_format : "ms", print_shape != 0);
        if (cap > 0) {
            size_t n = std::min<size_t>((size_t)cap - 1, r.size());
            std::memcpy(buf, r.data(), n);
            buf[n] = 0;
        }
    });
}

// ------------------------------------------------------------------ Trainer ---------------

// save_checkpoint / save_checkpoint_with_optim (adam may be null), checkpoint.mojo:197-300
MTLH_API int32_t mtlh_checkpoint_save(void* m, void* a, const char* path, int32_t iter) {
    return guard([&] { save_checkpoint(path, *static_cast<Model*>(m), static_cast<Adam*>(a), iter); });
}
// load_checkpoint / load_checkpoint_with_optim (adam may be null), checkpoint.mojo:303-440
MTLH_API int32_t mtlh_checkpoint_load(void* m, void* a, const char* path, int32_t* iter, int32_t* has_optim) {
    return guard([&] {
        CheckpointInfo info = load_checkpoint(path, *static_cast<Model*>(m), static_cast<Adam*>(a));
        if (iter) *iter = info.iter;
        if (has_optim) *has_optim = info.has_optim_state ? 1 : 0;
    });
}
MTLH_API int32_t mtlh_trainer_create(void* m, void* a, int32_t use_graph, int64_t bucket_bytes, void** out) {
    return guard([&] { *out = new Trainer(*static_cast<Model*>(m), *static_cast<Adam*>(a), use_graph != 0, bucket_bytes); });
}
MTLH_API int32_t mtlh_trainer_destroy(void* t) {
    delete static_cast<Trainer*>(t);
    return MTL_OK;
}
MTLH_API int32_t mtlh_trainer_step(void* t, int32_t n_in, const float* const* inputs, float* loss) {
    return guard([&] {
        std::vector<const float*> in(inputs, inputs + n_in);
        *loss = static_cast<Trainer*>(t)->step(in);
    });
}
MTLH_API int32_t mtlh_trainer_step_async(void* t, int32_t n_in, const float* const* inputs, float* pinned_loss) {
    return guard([&] {
        std::vector<const float*> in(inputs, inputs + n_in);
        static_cast<Trainer*>(t)->step_async(in, pinned_loss);
    });
}
MTLH_API int32_t mtlh_trainer_set_label_input(void* t, int32_t input_index, int32_t num_classes) {
    return guard([&] { static_cast<Trainer*>(t)->set_label_input(input_index, num_classes); });
}
MTLH_API int32_t mtlh_trainer_set_exchange(void* t, int32_t on) {
    return guard([&] { static_cast<Trainer*>(t)->set_exchange(on != 0); });
}
MTLH_API int64_t mtlh_trainer_input_bytes(void* t) { return static_cast<Trainer*>(t)->input_bytes_per_step(); }
MTLH_API int32_t mtlh_trainer_graph_active(void* t) { return static_cast<Trainer*>(t)->graph_active() ? 1 : 0; }
