// One training step as the reference's examples write it (examples/mnist.mojo:92-104):
//     loss = model.forward(x, y); optim.zero_grad(); model.backward(); optim.step()
// enqueued without intermediate waits, optionally replayed from a captured CUDA graph, and with
// the data-parallel gradient exchange started per bucket as soon as a layer's parameter gradients
// are final, so that it overlaps the backward pass of the earlier layers.
#pragma once

#include "model.hpp"

namespace mantle {

class Trainer {
   public:
    // use_graph: capture the step on its second call and replay it afterwards.
    // bucket_bytes: gradient spans are exchanged once this many bytes are final (data parallel).
    Trainer(Model& model, Adam& adam, bool use_graph, int64_t bucket_bytes = 256 * 1024);
    ~Trainer();

    // Inputs are host pointers (pinned memory keeps the copy asynchronous).  Returns the loss of
    // this step after waiting for it.
    float step(const std::vector<const float*>& host_inputs);
    // Same, but only enqueues; the loss lands in *pinned_loss once the stream reaches it.
    void step_async(const std::vector<const float*>& host_inputs, float* pinned_loss);

    // Declares graph input `input_index`, shaped [B, num_classes], as one-hot targets that the CALLER
    // hands over as B fp32 class labels (what the reference's DataLoader yields, data/dataloader.mojo:135-189;
    // examples/mnist.mojo:92-97 expands them on the host every batch).  step() / step_async() then copy
    // B floats for this input and the one-hot rows are written on the device (mtl_one_hot_f32).
    void set_label_input(int input_index, int num_classes);
    // Bytes a step copies host -> device for its inputs (labels counted as labels).
    int64_t input_bytes_per_step() const;

    // Diagnostic: with the exchange off a data-parallel Trainer skips the all-reduce of the gradients
    // (every rank then trains on its own shard only -- NOT a valid training run).  Timing a step with and
    // without it separates the compute time of a rank from the exposed part of the communication.
    void set_exchange(bool on) { exchange_ = on; }

    int64_t steps() const { return steps_; }
    bool graph_active() const { return graphs_[0] || graphs_[1] || graphs_[2]; }

   private:
    void enqueue_body();
    int stage_inputs(const std::vector<const float*>& host_inputs);   // returns the staging slot used
    void place_inputs(int slot);
    static void node_done_thunk(void* self, int node);
    void node_done(int node);
    void flush_bucket(bool last = false);
    void map_final_nodes();
    bool fusion_mapped_ = false;
    bool exchange_ = true;

    Model& model_;
    Adam& adam_;
    bool use_graph_;
    int64_t bucket_bytes_;
    int world_ = 1;
    // One captured step per source of the inputs: staging buffer 0, staging buffer 1 (the placement of the
    // batch -- a device copy per input, one-hot rows for label inputs -- is part of those two graphs), and
    // inputs already resident in the arena.
    mtl_graph* graphs_[3] = {nullptr, nullptr, nullptr};
    float* stage_[2] = {nullptr, nullptr};  // device staging buffers for the inputs, used in turn
    int64_t stage_floats_ = 0;
    std::vector<int> label_classes_;        // per graph input: 0 = dense tensor, C = labels expanded to C classes
    int64_t host_floats(size_t input) const;  // floats the caller provides for an input
    int64_t staged_ = 0;
    float* own_loss_ = nullptr;         // pinned word used by step()
    int64_t steps_ = 0;
    // data-parallel bucketing: for every node, the trainable parameters whose gradient is final
    // once that node's backward has run
    std::vector<std::vector<int>> final_at_node_;
    int64_t pending_lo_ = -1, pending_hi_ = -1;  // pending span [lo, hi) in floats
};

}  // namespace mantle
