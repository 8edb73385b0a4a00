// Host-side mirror of Mantle's graph executor and optimizer on top of the C ABI:
//   Model   mantle/nn/model.mojo:61-395   (allocate, forward/inference/execute, backward)
//   Adam    mantle/nn/optim.mojo:51-149   (zero_grad, step, m/v state)
//   forward_op / backward_op              mantle/autograd/ops/ops.mojo:243-528
// Storage differs from the reference on purpose: instead of one host allocation per symbol
// (collection.mojo:175-200) all tensors live in one device arena, and the trainable parameters,
// their gradients and both Adam moments are each ONE contiguous fp32 span in the order of
// get_trainable_parameters (optim.mojo:27-44), so that the optimizer is a single kernel and the
// data-parallel gradient exchange is a single buffer.
#pragma once

#include <map>
#include <string>
#include <vector>

#include "graph.hpp"

namespace mantle {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

class Model {
   public:
    Model(mtl_ctx* ctx, const Graph& g, uint64_t init_seed = 42);
    ~Model();
    Model(const Model&) = delete;
    Model& operator=(const Model&) = delete;

    // model.mojo:82-99: inputs are HOST pointers in graph-declaration order; returns the loss.
    float forward(const std::vector<const float*>& host_inputs);
    // model.mojo:101-111: runs nodes up to the last graph output; copies outputs to host.
    void inference(const std::vector<const float*>& host_inputs, const std::vector<float*>& host_outputs);
    // model.mojo:173-330 with no upper gradients: seeds d(loss) = 1.
    void backward();

    // Split form used by the training pipeline: everything enqueued, nothing waited for.
    void copy_inputs_async(const std::vector<const float*>& pinned_inputs);
    void execute(int num_nodes);
    void backward_enqueue();
    float* loss_device() const;
    float* input_device(int i) const { return T(g_.inputs.at((size_t)i)); }

    // Parameters.tensors / Parameters.grads access (host copies).
    void get_tensor(int symbol_id, float* host_out) const;
    void set_tensor(int symbol_id, const float* host_in);
    void get_grad(int symbol_id, float* host_out) const;
    bool has_grad(int symbol_id) const { return grad_off_.count(symbol_id) != 0; }
    bool has_tensor(int symbol_id) const { return tensor_off_.count(symbol_id) != 0; }
    // Every symbol with storage, in Parameters.tensors order (inputs, parameters, node outputs).
    const std::vector<Symbol>& allocation_order() const { return alloc_order_; }
    TensorShape shape_of(int symbol_id) const;
    // Collection.set_zero on every gradient (optim.mojo:90-92).
    void zero_grads();

    // When on (default), the first gradient contribution a buffer receives in a backward pass
    // overwrites it and later ones add, which equals zero_grad() followed by accumulation without
    // touching the buffers twice; zero_grads() then only zeroes buffers no node writes.
    // Off: every contribution accumulates, exactly like backward_op (ops.mojo:405,463,498).
    void set_overwrite_first(bool on) { overwrite_first_ = on; ce_grad_fresh_ = false; }

    // Chain fusion (off by default).  On: a CONV2D whose only consumer is a RELU writes the RELU's
    // output directly (mtl_conv2d_fwd_act) and the RELU node is not run -- and when a MAXPOOL2D is the
    // RELU's only reader, the CONV2D writes the pooled values and indices (mtl_conv2d_fwd_act_pool) and
    // the RELU output is not written either; a MAXPOOL2D fed by a RELU
    // that nothing else reads performs that RELU's backward as well (mtl_maxpool2d_bwd_idx_act).
    // A CONV2D's operand gradients come from one mtl_conv2d_bwd_fused call (the bias gradient is then
    // summed in a different order: equal within rounding, not bitwise).
    // Every other tensor that IS written holds exactly the bits the unfused run writes; what is never
    // written is the CONV2D output (pre-activation) and the gradient of the RELU output.  Symbols
    // that are graph outputs or have other consumers are never fused away.
    void set_fusion(bool on);
    bool fusion() const { return fusion_; }

    // Per-node timing, the counterpart of PerfMetrics (mantle/autograd/perf_utils.mojo:60-236; the
    // reference's hook, model.mojo:397-400, is an empty stub).  While on, every node's forward and
    // backward call is bracketed on the device (mtl_prof_range_*), so a node's time is the device time
    // of all kernels it launched -- not host time as in the reference.  Nodes a fused call computes
    // (a RELU run by its CONV2D, the loss chain) show zero; their time is in the node at the head of
    // the chain.  Steps replayed from a captured graph are not seen: profile with an eager Trainer
    // (use_graph = false) or with Model.forward / backward.
    void set_profiling(bool on);
    struct NodePerf { double fwd_ms = 0, bwd_ms = 0; int64_t fwd_launches = 0, bwd_launches = 0; };
    // Sums over the passes recorded since profiling was switched on; *passes = forward / backward passes seen.
    std::vector<NodePerf> perf_metrics(int* fwd_passes, int* bwd_passes);
    // The table PerfMetrics.print_perf_metrics prints: Node | Operator | Time [unit] | Percentage [%]
    // (| shapes), time = mean per pass.  time_format: "ns", "ms" or "s".
    std::string perf_report(bool forward, const std::string& time_format, bool print_shape);

    // flat trainable spans (device pointers) for the optimizer and the gradient exchange
    float* params_flat() const { return tensors_; }
    float* grads_flat() const { return grads_; }
    int64_t n_trainable() const { return n_trainable_; }
    const std::vector<Symbol>& trainable_parameters() const { return trainable_; }
    // Offsets (in floats) inside the flat spans, in trainable_parameters() order.
    const std::vector<int64_t>& trainable_offsets() const { return trainable_off_; }

    mtl_ctx* ctx() const { return ctx_; }
    const Graph& graph() const { return g_; }
    int n_inference_nodes() const { return n_inference_nodes_; }

    // The node during whose backward call the operand gradients of `node` are written: the node itself,
    // or -- for the bias ADD of a fused Linear layer -- the DOT node in front of it.
    int backward_performed_at(int node) const {
        return (fusion_ && (size_t)node < lin_dot_of_.size() && lin_dot_of_[(size_t)node] >= 0) ? lin_dot_of_[(size_t)node] : node;
    }

    // Called between backward nodes by the data-parallel trainer: node index (reverse order) done.
    void (*after_backward_node)(void* user, int node_index) = nullptr;
    void* after_backward_user = nullptr;

   private:
    void forward_op(const Node& n);
    void backward_op(const Node& n, int tensor_id);
    void refresh_pow_exponent(const Node& n);
    float* T(const Symbol& s) const;
    float* G(const Symbol& s) const;
    int acc_flag(const Symbol& s);
    const float* twin_of(const Symbol& s) const;  // valid channels-last twin of a tensor, or null
    void check(int rc, const char* what) const;

    mtl_ctx* ctx_;
    Graph g_;
    float* tensors_ = nullptr;  // arena: [trainable params | everything else]
    float* grads_ = nullptr;    // arena: [trainable param grads | other trainable symbols]
    int64_t n_tensor_floats_ = 0, n_grad_floats_ = 0, n_trainable_ = 0;
    std::map<int, int64_t> tensor_off_, grad_off_;
    std::map<int, TensorShape> shapes_;
    std::map<int, float> scalar_values_;      // host copies of [1]-shaped literals (POW exponent)
    std::map<int, int32_t*> pool_idx_;         // hidden argmax buffers, keyed by node index
    std::vector<Symbol> trainable_;
    std::vector<Symbol> alloc_order_;
    std::vector<int64_t> trainable_off_;
    std::map<int, int> alias_of_;              // result symbol of a copy node -> the operand whose storage it shares
    std::vector<char> alias_node_;             // copy nodes that move no data
    std::map<int, bool> grad_written_;
    std::vector<int> never_written_;           // trainable symbols no backward node writes
    bool overwrite_first_ = true;
    int n_inference_nodes_ = 0;
    bool fusion_ = false;
    bool profiling_ = false;
    int fwd_passes_ = 0, bwd_passes_ = 0;
    int ce_head_ = -1;                 // first of the nine nodes of a CrossEntropyLoss run as one call each way, or -1
    bool ce_sole_reader_ = false;      // the loss chain is the only reader of its logits
    bool ce_grad_fresh_ = false;       // the last forward pass left the logits' gradient in place
    int ce_scale_sym_ = -1;            // id of the [1]-shaped literal the loss is scaled by
    std::vector<int> fwd_relu_of_;     // per node: the RELU node a CONV2D also computes, or -1
    std::vector<int> fwd_pool_of_;     // per node: the MAXPOOL2D node a CONV2D+RELU also computes, or -1
    std::vector<char> fwd_skip_;       // RELU nodes computed by their producer
    std::vector<int> bwd_relu_of_;     // per node: the RELU node whose backward a MAXPOOL2D also performs, or -1
    std::vector<char> bwd_skip_;       // RELU nodes whose backward their consumer performs
    std::vector<int> bwd_pooled_of_;   // per CONV2D node: the MAXPOOL2D whose pooled gradient it consumes directly, or -1
    std::vector<char> bwd_pool_skip_;  // MAXPOOL2D nodes whose backward that CONV2D performs
    std::map<int, float*> twins_;      // channels-last copies of pooled outputs that feed a CONV2D, by symbol id
    std::map<int, bool> twin_valid_;   // written by the producing call of this step and not overwritten since
    std::vector<char> relu_in_absent_; // RELU nodes whose input tensor is not written (use the output as mask)
    std::vector<int> lin_add_of_;      // per DOT node: the ADD(bias) node that one mtl_linear_* call also covers, or -1
    std::vector<int> lin_dot_of_;      // per ADD node: the DOT node whose call covers it, or -1
};

class Adam {
   public:
    // optim.mojo:66-88
    Adam(Model& model, float lr = 0.001f, float beta1 = 0.9f, float beta2 = 0.999f, float epsilon = 1e-8f);
    ~Adam();
    void zero_grad() { model_.zero_grads(); }  // optim.mojo:90-92
    void step();                               // optim.mojo:94-140
    // Variant whose iteration counter lives on the device, for captured steps.
    void step_captured();
    // A captured step that is replayed advances the device counter; this keeps the host copy equal.
    void note_replayed_step() { iter_ += 1; }
    int iter() const { return iter_; }
    void set_grad_scale(float s) { grad_scale_ = s; }
    void get_state(int which /*0 m, 1 v*/, float* host_out) const;
    void set_state(int which /*0 m, 1 v*/, const float* host_in);
    // Continue from a stored step count (host and device copies of the counter).
    void set_iter(int iter);

   private:
    Model& model_;
    float lr_, beta1_, beta2_, eps_;
    int iter_ = 0;
    float grad_scale_ = 1.0f;
    float* m_ = nullptr;
    float* v_ = nullptr;
    int32_t* t_dev_ = nullptr;
};

}  // namespace mantle
