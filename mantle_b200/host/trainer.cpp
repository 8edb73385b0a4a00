#include "trainer.hpp"

#include <algorithm>

namespace mantle {

namespace {
void ck(mtl_ctx* ctx, int rc, const char* what) {
    if (rc != MTL_OK) throw Error(rc, std::string(what) + ": " + mtl_last_error(ctx));
}
}  // namespace

Trainer::Trainer(Model& model, Adam& adam, bool use_graph, int64_t bucket_bytes)
    : model_(model), adam_(adam), use_graph_(use_graph), bucket_bytes_(bucket_bytes) {
    mtl_ctx* ctx = model_.ctx();
    world_ = mtl_dp_world_size(ctx);
    ck(ctx, mtl_host_alloc(ctx, 64, (void**)&own_loss_), "pinned loss word");
    if (world_ > 1) adam_.set_grad_scale(1.0f / (float)world_);
    map_final_nodes();
    model_.after_backward_node = &Trainer::node_done_thunk;
    model_.after_backward_user = this;
}

// A parameter's gradient is final after the lowest-numbered node that reads it has run its backward
// (nodes run in reverse order) -- or, with chain fusion, after the node whose call writes it.
void Trainer::map_final_nodes() {
    const Graph& g = model_.graph();
    final_at_node_.assign(g.nodes.size(), {});
    const auto& tr = model_.trainable_parameters();
    for (size_t p = 0; p < tr.size(); ++p) {
        int first = -1;
        for (size_t i = 0; i < g.nodes.size() && first < 0; ++i)
            for (auto& in : g.nodes[i].inputs)
                if (in.id == tr[p].id) first = (int)i;
        if (first >= 0) final_at_node_[(size_t)model_.backward_performed_at(first)].push_back((int)p);
    }
    fusion_mapped_ = model_.fusion();
}

Trainer::~Trainer() {
    model_.after_backward_node = nullptr;
    model_.after_backward_user = nullptr;
    for (mtl_graph* g : graphs_)
        if (g) mtl_graph_destroy(model_.ctx(), g);
    for (int b = 0; b < 2; ++b)
        if (stage_[b]) mtl_free(model_.ctx(), stage_[b]);
    mtl_host_free(model_.ctx(), own_loss_);
}

void Trainer::set_label_input(int input_index, int num_classes) {
    const Graph& g = model_.graph();
    if (input_index < 0 || (size_t)input_index >= g.inputs.size()) throw Error(MTL_ERR_INVALID, "no such graph input");
    const TensorShape& s = g.inputs[(size_t)input_index].shape;
    if (s.rank != 2 || s[1] != num_classes || num_classes < 1)
        throw Error(MTL_ERR_INVALID, "a label input must be shaped [B, num_classes]");
    if (stage_[0]) throw Error(MTL_ERR_INVALID, "declare label inputs before the first step");
    label_classes_.resize(g.inputs.size(), 0);
    label_classes_[(size_t)input_index] = num_classes;
}

int64_t Trainer::host_floats(size_t i) const {
    const TensorShape& s = model_.graph().inputs[i].shape;
    return (i < label_classes_.size() && label_classes_[i]) ? s[0] : s.num_elements();
}

int64_t Trainer::input_bytes_per_step() const {
    int64_t n = 0;
    for (size_t i = 0; i < model_.graph().inputs.size(); ++i) n += host_floats(i) * 4;
    return n;
}

void Trainer::node_done_thunk(void* self, int node) { static_cast<Trainer*>(self)->node_done(node); }

// `last`: the bucket that ends the backward pass, which nothing can overlap: exchanged directly between the
// GPUs on the compute stream when the group can (mtl_dp_allreduce_tail), else like the others.
void Trainer::flush_bucket(bool last) {
    if (pending_lo_ < 0) return;
    float* span = model_.grads_flat() + pending_lo_;
    const int64_t n = pending_hi_ - pending_lo_;
    ck(model_.ctx(), last ? mtl_dp_allreduce_tail(model_.ctx(), span, n) : mtl_dp_allreduce_async(model_.ctx(), span, n),
       "gradient allreduce");
    pending_lo_ = pending_hi_ = -1;
}

void Trainer::node_done(int node) {
    if (world_ <= 1 || !exchange_) return;
    const auto& tr = model_.trainable_parameters();
    const auto& off = model_.trainable_offsets();
    for (int p : final_at_node_[node]) {
        int64_t lo = off[p];
        int64_t hi = (size_t)p + 1 < off.size() ? off[p + 1] : model_.n_trainable();
        (void)tr;
        if (pending_lo_ < 0) {
            pending_lo_ = lo;
            pending_hi_ = hi;
        } else if (hi == pending_lo_) {
            pending_lo_ = lo;  // grows downwards: backward visits parameters from last to first
        } else if (lo == pending_hi_) {
            pending_hi_ = hi;
        } else {
            flush_bucket();
            pending_lo_ = lo;
            pending_hi_ = hi;
        }
    }
    if (pending_lo_ >= 0 && (pending_hi_ - pending_lo_) * 4 >= bucket_bytes_) flush_bucket();
    if (node == 0) {
        flush_bucket(true);
        ck(model_.ctx(), mtl_dp_wait(model_.ctx()), "gradient allreduce wait");
    }
}

void Trainer::enqueue_body() {
    if (fusion_mapped_ != model_.fusion()) map_final_nodes();   // fusion was switched after construction
    model_.execute((int)model_.graph().nodes.size());
    adam_.zero_grad();
    model_.backward_enqueue();
    adam_.step_captured();
}

// Inputs travel host -> staging buffer on the copy stream (two buffers, used in turn) and staging
// buffer -> input tensors on the compute stream at the head of the step, so a caller that enqueues
// step i + 1 while step i is still running gets its copy overlapped with that step's kernels.
int Trainer::stage_inputs(const std::vector<const float*>& host_inputs) {
    mtl_ctx* ctx = model_.ctx();
    const Graph& g = model_.graph();
    if (host_inputs.size() != g.inputs.size()) throw Error(MTL_ERR_INVALID, "wrong number of inputs");
    if (!stage_[0]) {
        stage_floats_ = 0;
        for (size_t i = 0; i < g.inputs.size(); ++i) stage_floats_ += (host_floats(i) + 63) / 64 * 64;
        for (int b = 0; b < 2; ++b)
            ck(ctx, mtl_malloc(ctx, (size_t)std::max<int64_t>(stage_floats_, 64) * 4, (void**)&stage_[b]), "input staging buffer");
    }
    const int slot = (int)(staged_ & 1);
    ++staged_;
    int64_t off = 0;
    for (size_t i = 0; i < host_inputs.size(); ++i) {
        const int64_t n = host_floats(i);
        ck(ctx, mtl_stage_h2d(ctx, slot, stage_[slot] + off, host_inputs[i], (size_t)n * 4), "input copy");
        off += (n + 63) / 64 * 64;
    }
    ck(ctx, mtl_stage_acquire(ctx, slot), "input copy wait");
    return slot;
}

// Staging buffer -> input tensors (a device copy; one-hot rows for an input declared with set_label_input).
// Enqueued on the compute stream; inside a capture it becomes part of that slot's graph.
void Trainer::place_inputs(int slot) {
    mtl_ctx* ctx = model_.ctx();
    const Graph& g = model_.graph();
    int64_t off = 0;
    for (size_t i = 0; i < g.inputs.size(); ++i) {
        const int64_t n = host_floats(i);
        if (i < label_classes_.size() && label_classes_[i])
            ck(ctx, mtl_one_hot_f32(ctx, model_.input_device((int)i), stage_[slot] + off, n, label_classes_[i]),
               "one-hot targets");
        else
            ck(ctx, mtl_copy_f32(ctx, model_.input_device((int)i), stage_[slot] + off, n, 0), "input placement");
        off += (n + 63) / 64 * 64;
    }
}

void Trainer::step_async(const std::vector<const float*>& host_inputs, float* pinned_loss) {
    mtl_ctx* ctx = model_.ctx();
    // which captured step this is: inputs from staging buffer 0 / 1, or already resident (2)
    const int variant = host_inputs.empty() ? 2 : stage_inputs(host_inputs);
    ++steps_;
    if (!use_graph_ || steps_ == 1) {
        // the first step also sizes the scratch workspace, which must not grow during capture
        if (variant < 2) place_inputs(variant);
        enqueue_body();
    } else {
        if (!graphs_[variant]) {
            ck(ctx, mtl_graph_begin(ctx), "graph capture begin");
            try {
                if (variant < 2) place_inputs(variant);
                enqueue_body();
            } catch (...) {
                mtl_graph* dead = nullptr;
                mtl_graph_end(ctx, &dead);
                if (dead) mtl_graph_destroy(ctx, dead);
                throw;
            }
            ck(ctx, mtl_graph_end(ctx, &graphs_[variant]), "graph capture end");
        } else {
            adam_.note_replayed_step();
        }
        ck(ctx, mtl_graph_launch(ctx, graphs_[variant]), "graph launch");
    }
    // the staging buffer may be overwritten once the step that read it is over
    if (variant < 2) ck(ctx, mtl_stage_release(ctx, variant), "input staging release");
    // the loss tensor is not touched by the backward pass, so it is read after the whole step
    ck(ctx, mtl_d2h_async(ctx, pinned_loss, model_.loss_device(), 4), "loss read-back");
}

float Trainer::step(const std::vector<const float*>& host_inputs) {
    step_async(host_inputs, own_loss_);
    ck(model_.ctx(), mtl_sync(model_.ctx()), "step wait");
    return *own_loss_;
}

}  // namespace mantle
