/*
 * mantle_cuda.h -- C ABI of libmantle_cuda.so, the B200 (sm_100a) execution backend for
 * Mantle's operator registry.
 *
 * Mantle dispatches every graph node through
 *     forward_op [op, shapes..., attrs](res, t1[, t2[, t3]])        mantle/autograd/ops/ops.mojo:243-352
 *     backward_op[tensor_id, op, ug_shape, shapes..., attrs](ug, t1[, t2[, t3]], grad)
 *                                                                    mantle/autograd/ops/ops.mojo:355-528
 * and updates weights with Adam.step / Adam.zero_grad               mantle/nn/optim.mojo:90-140.
 * Each arm of those dispatchers maps to exactly one entry point below; the comment above an entry
 * point names the reference function it replaces.  Op ids are the reference's OP.* ids
 * (mantle/autograd/ops/ops.mojo:57-83).
 *
 * Conventions
 *   - every function returns an int32 status (MTL_OK == 0); the text of the last error of a
 *     context is available through mtl_last_error().  Nothing aborts and no kernel traps.
 *   - all tensor pointers are DEVICE pointers to dense row-major fp32 data unless the parameter
 *     is documented as host memory; shapes are host integers.
 *   - calls on one context are enqueued on that context's stream in call order and return
 *     without waiting for the GPU (mtl_d2h and mtl_sync wait).
 *   - one context is driven by one host thread at a time; different contexts are independent.
 *   - backward entry points take `accumulate`: non-zero adds the contribution to `grad`
 *     (the reference's accumulate_grad, mantle/core/tensorutils.mojo:443-487), zero overwrites.
 *   - there is no CPU fallback: without a usable CUDA device mtl_ctx_create fails.
 */
#ifndef MANTLE_CUDA_H_
#define MANTLE_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MTL_API __attribute__((visibility("default")))
#else
#define MTL_API
#endif

typedef struct mtl_ctx mtl_ctx;
typedef struct mtl_graph mtl_graph;

#define MTL_MAX_RANK 8 /* TensorShape rank limit, mantle/core/tensor.mojo */

enum mtl_status {
    MTL_OK = 0,
    MTL_ERR_INVALID = 1,     /* bad argument: null pointer, bad shape, unknown op id        */
    MTL_ERR_CUDA = 2,        /* a CUDA runtime / driver call failed                          */
    MTL_ERR_UNSUPPORTED = 3, /* valid in the reference but outside this backend's coverage   */
    MTL_ERR_NOMEM = 4,       /* device allocation failed, or workspace growth while capturing */
    MTL_ERR_TIMEOUT = 5,     /* a bounded device-side wait ran out (kernel returned cleanly)  */
    MTL_ERR_COMM = 6         /* collective library error                                     */
};

/* Arithmetic used by OP.DOT and OP.CONV2D.
 *   MTL_MATH_FP32   CUDA-core fp32 FMA chains in ascending k, bit-identical to the reference's
 *                   per-element accumulation in matmul.mojo:50-62 for DOT.
 *   MTL_MATH_TF32   tcgen05 kind::tf32 tensor-core GEMM, fp32 accumulate in TMEM.
 *   MTL_MATH_TF32X3 each operand split into tf32 hi + lo parts, three tensor-core products
 *                   (hi*hi + hi*lo + lo*hi); fp32-faithful results.
 * Shapes the tensor-core kernels cannot take (unaligned strides, tiny extents) run on the
 * CUDA-core kernels in every mode. */
enum mtl_math_mode { MTL_MATH_FP32 = 0, MTL_MATH_TF32 = 1, MTL_MATH_TF32X3 = 2 };

/* OP.* ids accepted by the generic entry points (mantle/autograd/ops/ops.mojo:57-83). */
enum mtl_op {
    MTL_OP_ADD = 0, MTL_OP_SUB = 1, MTL_OP_MUL = 2, MTL_OP_DIV = 3,
    MTL_OP_EXP = 4, MTL_OP_LOG = 5, MTL_OP_POW = 6, MTL_OP_DOT = 7,
    MTL_OP_SUM = 8, MTL_OP_MEAN = 9, MTL_OP_MAX = 10,
    MTL_OP_FLATTEN = 11, MTL_OP_RESHAPE = 12,
    MTL_OP_SIGMOID = 13, MTL_OP_RELU = 14, MTL_OP_TANH = 15,
    MTL_OP_CONV2D = 16, MTL_OP_TRANSPOSE = 17, MTL_OP_MAXPOOL2D = 18, MTL_OP_FMA = 19,
    MTL_OP_CLIP = 20, MTL_OP_SQUEEZE = 21, MTL_OP_UNSQUEEZE = 22,
    MTL_OP_CONCAT = 23, MTL_OP_SPLIT = 24, MTL_OP_SLICE = 25,
    MTL_OP_LEAKYRELU = 28
};

/* ---------------------------------------------------------------- lifecycle ------------- */

/* Creates a context on CUDA device `device` with its own non-blocking stream.
 * Replaces nothing in the reference (which has no device); it is the handle every op needs. */
MTL_API int32_t mtl_ctx_create(int32_t device, mtl_ctx** out);
MTL_API int32_t mtl_ctx_destroy(mtl_ctx* ctx);
/* Use an existing cudaStream_t (passed as void*) instead of the context's own stream. */
MTL_API int32_t mtl_ctx_set_stream(mtl_ctx* ctx, void* cuda_stream);
MTL_API void*   mtl_ctx_stream(mtl_ctx* ctx);
MTL_API int32_t mtl_ctx_set_math_mode(mtl_ctx* ctx, int32_t mode);
MTL_API int32_t mtl_ctx_math_mode(mtl_ctx* ctx);
/* Pre-sizes the internal scratch workspace (operand splits, channels-last staging, split-K
 * partials).  It grows on demand outside stream capture; growth during capture is an error. */
MTL_API int32_t mtl_ctx_reserve_workspace(mtl_ctx* ctx, size_t bytes);
/* State of that workspace (any out pointer may be null): its size and address, the number of
 * instantiated graphs (mtl_graph_end) still alive on the context, and the number of older
 * workspace blocks kept because such a graph was captured with them.  A block that has to grow
 * while graphs are alive is not freed -- a replayed step goes on using the block it was captured
 * with -- and is released when the last graph is destroyed.  No counterpart in the reference. */
MTL_API int32_t mtl_ctx_workspace_info(mtl_ctx* ctx, size_t* bytes, void** block, int32_t* live_graphs,
                                       int32_t* retired_blocks);
MTL_API int32_t mtl_sync(mtl_ctx* ctx);
MTL_API const char* mtl_last_error(mtl_ctx* ctx);
/* Number of kernels this library launched on the context since creation (memsets and copies
 * are not counted). */
MTL_API int64_t mtl_launch_count(mtl_ctx* ctx);
/* Tiles of the implicit-GEMM convolution kernels that were split along the reduction over two
 * CTAs (the tiles of a partial last wave), summed over every launch of the context so far; -1
 * without a context.  A diagnostic: tests use it to know that the split path ran.  No counterpart
 * in the reference. */
MTL_API int64_t mtl_conv_split_tiles(mtl_ctx* ctx);
/* Reads and clears the device-side status word that bounded waits write on time-out. */
MTL_API int32_t mtl_device_status(mtl_ctx* ctx, int32_t* out_status);
MTL_API const char* mtl_version(void);
/* Self-test of the bounded device-side wait: launches one small kernel that waits, for at most
 * budget_us microseconds, on a barrier nothing will ever complete.  The wait gives up, the kernel
 * writes MTL_ERR_TIMEOUT to the status word that mtl_device_status reads (and clears) and returns;
 * the context stays usable.  *waited_us (may be null) receives how long the kernel waited.  It shows
 * that a lost completion inside a tensor-core kernel ends as a status code, not as a hung GPU. */
MTL_API int32_t mtl_selftest_bounded_wait(mtl_ctx* ctx, int32_t budget_us, int32_t* waited_us);

/* ---------------------------------------------------------------- memory ---------------- */

/* Device storage behind Collection / Parameters (mantle/autograd/collection.mojo:175-222). */
MTL_API int32_t mtl_malloc(mtl_ctx* ctx, size_t bytes, void** out_dptr);
MTL_API int32_t mtl_free(mtl_ctx* ctx, void* dptr);
/* Debug aid, no counterpart in the reference.  With MANTLE_CUDA_DEBUG=1 in the environment when a
 * context is created, every mtl_malloc block sits between two 256-byte guard zones filled with a
 * byte pattern; mtl_debug_check (also run by mtl_sync and mtl_free in that mode) waits for the
 * stream and verifies them, returning MTL_ERR_INVALID with a message that names the damaged block,
 * the side and the distance of the stray write.  Without the variable it returns MTL_OK at once. */
MTL_API int32_t mtl_debug_check(mtl_ctx* ctx);
/* Model.execute step 1, inputs into the arena (mantle/nn/model.mojo:117-119); src is host. */
MTL_API int32_t mtl_h2d(mtl_ctx* ctx, void* dst, const void* src_host, size_t bytes);
/* Model.forward's return / Model.inference's copies (model.mojo:99,108-110); dst is host;
 * waits for the stream. */
MTL_API int32_t mtl_d2h(mtl_ctx* ctx, void* dst_host, const void* src, size_t bytes);
/* Staged input copies on a second stream, so that the host-to-device copy of the next batch runs
 * while the current step computes (no counterpart in the reference, whose Model.forward copies its
 * inputs synchronously, model.mojo:117-119).  `slot` is 0..3; each slot stands for one staging buffer
 * owned by the caller.
 *   mtl_stage_h2d      copies on the copy stream once the compute stream has released the slot
 *   mtl_stage_acquire  makes the compute stream wait for everything staged into the slot so far
 *   mtl_stage_release  marks, on the compute stream, that the slot may be overwritten */
MTL_API int32_t mtl_stage_h2d(mtl_ctx* ctx, int32_t slot, void* dst_dev, const void* src_host, size_t bytes);
MTL_API int32_t mtl_stage_acquire(mtl_ctx* ctx, int32_t slot);
MTL_API int32_t mtl_stage_release(mtl_ctx* ctx, int32_t slot);

/* Asynchronous variants for pinned host memory (see mtl_host_alloc). */
MTL_API int32_t mtl_h2d_async(mtl_ctx* ctx, void* dst, const void* src_host, size_t bytes);
MTL_API int32_t mtl_d2h_async(mtl_ctx* ctx, void* dst_host, const void* src, size_t bytes);
MTL_API int32_t mtl_host_alloc(mtl_ctx* ctx, size_t bytes, void** out_hptr);
MTL_API int32_t mtl_host_free(mtl_ctx* ctx, void* hptr);
/* Collection.set_zero (collection.mojo:222) and fill (mantle/core/tensorutils.mojo:30-44). */
MTL_API int32_t mtl_zero(mtl_ctx* ctx, void* dptr, size_t bytes);
MTL_API int32_t mtl_fill_f32(mtl_ctx* ctx, float* dptr, int64_t n, float value);
/* One-hot targets on the device: out[b][c] = 1 when c == Int(labels[b]) else 0, for fp32 class labels as the
 * reference's DataLoader hands them over (examples/mnist.mojo:92-97 builds this tensor on the host every
 * batch).  The step then copies B floats of labels instead of B*C floats of targets.  A label outside
 * [0, C) gives an all-zero row (the reference would write outside the row). */
MTL_API int32_t mtl_one_hot_f32(mtl_ctx* ctx, float* out, const float* labels, int64_t B, int64_t C);
/* RESHAPE / FLATTEN / SQUEEZE / UNSQUEEZE forward and backward are copies
 * (mantle/autograd/ops/basics.mojo:706-756, mlops.mojo:302-373). accumulate != 0: dst += src. */
MTL_API int32_t mtl_copy_f32(mtl_ctx* ctx, float* dst, const float* src, int64_t n,
                             int32_t accumulate);

/* ---------------------------------------------------------------- DOT ------------------- */

/* DOT.forward -> dot (basics.mojo:230-237, matmul.mojo:80-153): C[M,N] = A[M,K] . B[K,N]. */
MTL_API int32_t mtl_dot_fwd(mtl_ctx* ctx, float* C, const float* A, const float* B,
                            int64_t M, int64_t K, int64_t N);
/* DOT.backward (basics.mojo:240-257): tensor_id 0: grad[M,K] (+)= ug[M,N] . B^T
 * (dot_transpose_t2, matmul.mojo:175-182); tensor_id 1: grad[K,N] (+)= A^T . ug
 * (dot_transpose_t1, matmul.mojo:203-210).  The operand not needed may be null. */
MTL_API int32_t mtl_dot_bwd(mtl_ctx* ctx, int32_t tensor_id, float* grad, const float* ug,
                            const float* A, const float* B, int64_t M, int64_t K, int64_t N,
                            int32_t accumulate);

/* nn.Linear, i.e. the DOT node and the ADD of the bias that follows it (mantle/nn/layers/linear.mojo:25-46),
 * as one call each way.  No single counterpart in the reference: each call gives the result of the
 * reference's operator calls named below.
 *   mtl_linear_fwd   C[M,N] = A[M,K] . B[K,N] + bias[N]: DOT.forward (basics.mojo:230-237) followed by
 *                    ADD.forward with the bias broadcast over the rows (basics.mojo:21-43); bias may be null.
 *   mtl_linear_bwd   from the upper gradient ug[M,N] of the ADD's result: dA (+)= ug . B^T and
 *                    dB (+)= A^T . ug (DOT.backward, basics.mojo:240-257), dbias (+)= column sums of ug
 *                    (ADD.backward with un-broadcasting, basics.mojo:46-66, tensorutils.mojo:455-487).  Any of
 *                    dA, dB, dbias may be null; each has its own accumulate flag.
 * For N <= 16 outside MTL_MATH_FP32 each call is ONE launch: the sums over k (forward) and over the
 * batch (dB) are cut into slices, and the block that finishes last for a group of rows folds the slices
 * in ascending order, so the result does not depend on scheduling (fp32 FMA on CUDA cores; the sums
 * are re-associated with respect to the reference's chain, within rtol = atol = 1e-5).  Other shapes
 * and MTL_MATH_FP32 run the separate operator entry points. */
MTL_API int32_t mtl_linear_fwd(mtl_ctx* ctx, float* C, const float* A, const float* B, const float* bias,
                               int64_t M, int64_t K, int64_t N);
MTL_API int32_t mtl_linear_bwd(mtl_ctx* ctx, float* dA, float* dB, float* dbias, const float* ug,
                               const float* A, const float* B, int64_t M, int64_t K, int64_t N,
                               int32_t acc_da, int32_t acc_db, int32_t acc_dbias);

/* ---------------------------------------------------------------- CONV2D ---------------- */

/* Geometry shared by the convolution and pooling entry points; the index lists are the
 * reference's "padding", "stride", "dilation" attributes (x = dim -2, y = dim -1). */
typedef struct mtl_conv2d_desc {
    int32_t N, C, H, W; /* inputs  [N, C, H, W]                                   */
    int32_t K, R, S;    /* kernel  [K, C, R, S]; for pooling K is ignored, R,S = kernel_size */
    int32_t pad[2], stride[2], dilation[2];
} mtl_conv2d_desc;

/* get_result_shape (mantle/autograd/ops/conv.mojo:25-58). Host-only helper. */
MTL_API int32_t mtl_conv2d_out_shape(const mtl_conv2d_desc* d, int32_t* OH, int32_t* OW);
/* CONV2D.forward (conv.mojo:81-226): Y[N,K,OH,OW] = conv(X, Wt) + bias[K]. */
MTL_API int32_t mtl_conv2d_fwd(mtl_ctx* ctx, float* Y, const float* X, const float* Wt,
                               const float* bias, const mtl_conv2d_desc* d);
/* CONV2D.backward (conv.mojo:229-425): tensor_id 0 -> grad = dX, 1 -> dW, 2 -> dbias. */
MTL_API int32_t mtl_conv2d_bwd(mtl_ctx* ctx, int32_t tensor_id, float* grad, const float* ug,
                               const float* X, const float* Wt, const mtl_conv2d_desc* d,
                               int32_t accumulate);

/* ---------------------------------------------------------------- MAXPOOL2D ------------- */

/* MAXPOOL2D.forward (mantle/autograd/ops/pool.mojo:44-100).  `idx` (may be null) receives for
 * every output element the plane-local input offset ih*W+iw of the first maximum in the
 * reference's (kx, ky) scan order under its strict `>` update; -1 when the window holds no
 * value greater than -inf. */
MTL_API int32_t mtl_maxpool2d_fwd(mtl_ctx* ctx, float* Y, int32_t* idx, const float* X,
                                  const mtl_conv2d_desc* d);
/* MAXPOOL2D.backward (pool.mojo:103-165): recomputes the argmax from X like the reference and
 * adds ug into dX at it.  Windows with no argmax (-1) contribute nothing; the reference writes
 * out of bounds there (pool.mojo:128,163). */
MTL_API int32_t mtl_maxpool2d_bwd(mtl_ctx* ctx, float* dX, const float* ug, const float* X,
                                  const mtl_conv2d_desc* d, int32_t accumulate);
/* Same result from the indices mtl_maxpool2d_fwd stored, without re-reading X. */
MTL_API int32_t mtl_maxpool2d_bwd_idx(mtl_ctx* ctx, float* dX, const float* ug,
                                      const int32_t* idx, const mtl_conv2d_desc* d,
                                      int32_t accumulate);

/* Fused forms for a CONV2D -> RELU -> MAXPOOL2D chain.  Neither has a single counterpart in the
 * reference: each gives exactly the result of two of its operator calls and lets the caller skip
 * one full-size tensor.  act_op is MTL_OP_RELU, or negative for "no activation".
 *   mtl_conv2d_fwd_act         Y = RELU.forward(CONV2D.forward(X, Wt, bias))  (conv.mojo:81-226 then
 *                              mlops.mojo RELU): the pre-activation tensor is never written.
 *   mtl_maxpool2d_bwd_idx_act  dX (+)= RELU.backward(MAXPOOL2D.backward(ug)), where dX is the gradient of
 *                              the RELU's INPUT and `pooled` the pooling output of the forward pass: the
 *                              element a window selected is the pooled value itself, so (pooled > 0) is
 *                              the RELU mask of the only element that receives a gradient. */
/*   mtl_conv2d_bwd_fused       CONV2D.backward for several operands in one call (conv.mojo:229-425): any of
 *                              dX, dW, db may be null (not wanted); each has its own accumulate flag.  The
 *                              gradients equal those of separate mtl_conv2d_bwd calls (db up to the order
 *                              of its sum); ug is re-laid out once and the bias gradient is read off
 *                              that pass. */
MTL_API int32_t mtl_conv2d_bwd_fused(mtl_ctx* ctx, float* dX, float* dW, float* db, const float* ug,
                                     const float* X, const float* Wt, const mtl_conv2d_desc* d,
                                     int32_t acc_dx, int32_t acc_dw, int32_t acc_db);
/*   mtl_conv2d_bwd_pooled      dX, dW, db (+)= CONV2D.backward of RELU.backward(MAXPOOL2D.backward(pooled_ug)): the
 *                              layer's gradients computed from the POOLED upper gradient, the argmax indices
 *                              and the pooled values, so the dense gradient of the layer's output (zero except
 *                              one element per window) is never written in NCHW: tensor-core layers scatter
 *                              it straight into their channels-last operand copy, the first-layer kernel
 *                              rebuilds it in shared memory; other geometries pass through scratch memory.
 *                              Any of dX, dW, db may be null; X_cl as in mtl_conv2d_bwd_fused_cl. */
MTL_API int32_t mtl_conv2d_bwd_pooled(mtl_ctx* ctx, float* dX, float* dW, float* db,
                                      const float* pooled_ug, const int32_t* idx, const float* pooled,
                                      const float* X, const float* X_cl, const float* Wt,
                                      const mtl_conv2d_desc* d, int32_t act_op,
                                      const mtl_conv2d_desc* pool, int32_t acc_dx, int32_t acc_dw,
                                      int32_t acc_db);
MTL_API int32_t mtl_conv2d_fwd_act(mtl_ctx* ctx, float* Y, const float* X, const float* Wt,
                                   const float* bias, const mtl_conv2d_desc* d, int32_t act_op);
/*   mtl_conv2d_fwd_act_pool    pooled, idx = MAXPOOL2D.forward(act(CONV2D.forward(X, Wt, bias))) (conv.mojo:81-226,
 *                              pool.mojo:44-100): `pool` describes the pooling of the convolution's output
 *                              (N, C = K, H = OH, W = OW, R/S = kernel_size).  Where a kernel pools in its
 *                              epilogue (2x2 windows, stride 2) the activation never reaches memory;
 *                              otherwise it passes through scratch memory.  idx may be null. */
MTL_API int32_t mtl_conv2d_fwd_act_pool(mtl_ctx* ctx, float* pooled, int32_t* idx, const float* X,
                                        const float* Wt, const float* bias,
                                        const mtl_conv2d_desc* d, int32_t act_op,
                                        const mtl_conv2d_desc* pool);
/* The same two calls with channels-last ([N, H, W, C]) twins, which the tensor-core convolution kernels
 * read: `pooled_cl` (may be null) receives a channels-last copy of the pooled output, written by the
 * kernel itself where it can and by one extra pass otherwise; `X_cl` (may be null) is such a copy of X
 * that the caller already holds (used in plain TF32 mode, where it replaces the call's own copy pass).
 * The caller owns both buffers and keeps X_cl equal to X. */
MTL_API int32_t mtl_conv2d_fwd_act_pool_cl(mtl_ctx* ctx, float* pooled, int32_t* idx, float* pooled_cl,
                                           const float* X, const float* X_cl, const float* Wt,
                                           const float* bias, const mtl_conv2d_desc* d, int32_t act_op,
                                           const mtl_conv2d_desc* pool);
MTL_API int32_t mtl_conv2d_bwd_fused_cl(mtl_ctx* ctx, float* dX, float* dW, float* db, const float* ug,
                                        const float* X, const float* X_cl, const float* Wt,
                                        const mtl_conv2d_desc* d, int32_t acc_dx, int32_t acc_dw,
                                        int32_t acc_db);
MTL_API int32_t mtl_maxpool2d_bwd_idx_act(mtl_ctx* ctx, float* dX, const float* ug,
                                          const int32_t* idx, const float* pooled,
                                          const mtl_conv2d_desc* d, int32_t act_op,
                                          int32_t accumulate);

/* ---------------------------------------------------------------- layout operators ------ */

/* TRANSPOSE.forward / .backward (mantle/autograd/ops/basics.mojo:618-703): out = permute(in, axes);
 * axes == NULL reverses the axes.  Backward adds the inverse permutation of ug to grad. */
MTL_API int32_t mtl_transpose_fwd(mtl_ctx* ctx, float* out, const float* in, int32_t rank,
                                  const int64_t* in_shape, const int32_t* axes);
MTL_API int32_t mtl_transpose_bwd(mtl_ctx* ctx, float* grad, const float* ug, int32_t rank,
                                  const int64_t* in_shape, const int32_t* axes, int32_t accumulate);

/* SLICE (mantle/autograd/ops/mlops.mojo:376-656): the reference's "starts", "ends", "steps", "axes"
 * attributes, n entries; axes[i] < 0 means axis i (its default).  Negative starts / ends count from
 * the end and are clamped to [0, dim] (adjust_boundary); steps may be negative.  A slice that is
 * empty or reaches outside the tensor is refused (the reference does not check). */
typedef struct mtl_slice_desc {
    int32_t n;
    int32_t axes[8];
    int64_t starts[8], ends[8], steps[8];
} mtl_slice_desc;
MTL_API int32_t mtl_slice_out_shape(int32_t rank, const int64_t* in_shape, const mtl_slice_desc* d,
                                    int64_t* out_shape);
MTL_API int32_t mtl_slice_fwd(mtl_ctx* ctx, float* out, const float* in, int32_t rank,
                              const int64_t* in_shape, const mtl_slice_desc* d);
MTL_API int32_t mtl_slice_bwd(mtl_ctx* ctx, float* grad, const float* ug, int32_t rank,
                              const int64_t* in_shape, const mtl_slice_desc* d, int32_t accumulate);

/* CONCAT / SPLIT (mantle/autograd/ops/dynamics.mojo:25-199) along axis `dim`.  in_shapes holds n_in
 * shapes of `rank` entries each; sections holds the n_out extents of the split axis. */
MTL_API int32_t mtl_concat_fwd(mtl_ctx* ctx, float* out, const float* const* ins, int32_t n_in,
                               int32_t rank, const int64_t* in_shapes, int32_t dim);
MTL_API int32_t mtl_concat_bwd(mtl_ctx* ctx, float* grad, const float* ug, int32_t input_id,
                               int32_t n_in, int32_t rank, const int64_t* in_shapes, int32_t dim,
                               int32_t accumulate);
MTL_API int32_t mtl_split_fwd(mtl_ctx* ctx, float* const* outs, const float* in, int32_t n_out,
                              int32_t rank, const int64_t* in_shape, const int64_t* sections,
                              int32_t dim);
MTL_API int32_t mtl_split_bwd(mtl_ctx* ctx, float* grad, const float* const* ugs, int32_t n_out,
                              int32_t rank, const int64_t* in_shape, const int64_t* sections,
                              int32_t dim, int32_t accumulate);

/* ---------------------------------------------------------------- elementwise ----------- */

/* ADD/SUB/MUL/DIV.forward -> elwise_op / broadcast_elwise_op (tensorutils.mojo:243-357):
 * scalar path when a shape is [1], NumPy broadcasting otherwise. out has the broadcast shape. */
MTL_API int32_t mtl_binary_fwd(mtl_ctx* ctx, int32_t op, float* out, const float* a,
                               const float* b, int32_t a_rank, const int64_t* a_shape,
                               int32_t b_rank, const int64_t* b_shape);
/* ADD/SUB/MUL/DIV.backward + un-broadcasting accumulate_grad (basics.mojo:46-219,
 * ops.mojo:457-463, tensorutils.mojo:455-487). ug has the broadcast shape. */
MTL_API int32_t mtl_binary_bwd(mtl_ctx* ctx, int32_t op, int32_t tensor_id, float* grad,
                               const float* ug, const float* a, const float* b,
                               int32_t a_rank, const int64_t* a_shape, int32_t b_rank,
                               const int64_t* b_shape, int32_t accumulate);
/* EXP, LOG, POW, SIGMOID, RELU, TANH, CLIP, LEAKYRELU forward (basics.mojo:260-327,
 * mlops.mojo:27-299).  p0/p1: POW exponent (truncated to int like elwise_pow) / unused;
 * LEAKYRELU negative_slope / unused; CLIP min / max. */
MTL_API int32_t mtl_unary_fwd(mtl_ctx* ctx, int32_t op, float* out, const float* in, int64_t n,
                              float p0, float p1);
/* Their backward arms; `in` is the forward INPUT (the reference differentiates at the input,
 * e.g. relu_bw mlops.mojo:94-100; POW uses a*(x+1e-12)^(a-1), basics.mojo:350-355). */
MTL_API int32_t mtl_unary_bwd(mtl_ctx* ctx, int32_t op, float* grad, const float* ug,
                              const float* in, int64_t n, float p0, float p1,
                              int32_t accumulate);
/* POW.backward for the exponent (tensor_id 1, basics.mojo:359-376): grad[0] (+)= sum over the n
 * elements of in^exponent * log(in) * ug, where log(in) counts as 0 when it is infinite (in == 0).
 * grad is the [1]-shaped gradient of the exponent; the sum runs as a two-pass tree. */
MTL_API int32_t mtl_pow_bwd_exponent(mtl_ctx* ctx, float* grad, const float* ug, const float* in,
                                     int64_t n, float exponent, int32_t accumulate);
/* FMA.forward/backward (basics.mojo:759-817): out = a*b + c, all the same shape. */
MTL_API int32_t mtl_fma_fwd(mtl_ctx* ctx, float* out, const float* a, const float* b,
                            const float* c, int64_t n);
MTL_API int32_t mtl_fma_bwd(mtl_ctx* ctx, int32_t tensor_id, float* grad, const float* ug,
                            const float* a, const float* b, int64_t n, int32_t accumulate);

/* ---------------------------------------------------------------- reductions ------------ */

/* SUM/MEAN/MAX.forward -> tsum/tmean/tmax (basics.mojo:381-534, tensorutils.mojo:565-876).
 * axis < 0 reduces everything to shape [1]; otherwise the axis keeps size 1. */
MTL_API int32_t mtl_reduce_fwd(mtl_ctx* ctx, int32_t op, float* out, const float* in,
                               int32_t rank, const int64_t* shape, int32_t axis);
/* SUM/MEAN/MAX.backward (basics.mojo:409-425, 455-506, 537-615); MAX splits the gradient
 * 1/n between n tied maxima. */
MTL_API int32_t mtl_reduce_bwd(mtl_ctx* ctx, int32_t op, float* grad, const float* ug,
                               const float* in, int32_t rank, const int64_t* shape,
                               int32_t axis, int32_t accumulate);

/* Whole-tensor SUM / MEAN / MAX that performs no allocation of any kind.
 * No counterpart in the reference: it exists for hosts that must not allocate device memory at
 * the moment they reduce -- for example an embedding whose GPU memory has been handed out in full
 * to another pool at start-up, so that a cudaMalloc would fail, or a service loop that may not
 * take the implicit device-wide wait an allocation can bring.  mtl_reduce_fwd keeps its per-block
 * partial results in the context's growable workspace; this variant keeps them in a fixed array
 * compiled into the library (4 KB, held by every GPU that loads the library until exit) and
 * therefore accepts at most MTL_REDUCE_STATIC_MAX_ELEMENTS elements; larger sizes are rejected
 * with MTL_ERR_INVALID.  Results equal mtl_reduce_fwd(op, out, in, 1, {n}, -1).
 * The first call on a device looks up the array's device address (no allocation); make that call
 * before starting a stream capture (inside mtl_graph_begin/_end a first call is refused with
 * MTL_ERR_INVALID).  Like every entry point it runs with the context's device current and leaves the
 * caller's current device as it found it.  All calls on a device share the one array: two calls whose
 * kernels overlap on the GPU (different streams or contexts) race and give wrong results; calls
 * on one stream are ordered and safe. */
#define MTL_REDUCE_STATIC_MAX_ELEMENTS (1ll << 28)
MTL_API int32_t mtl_reduce_all_static(mtl_ctx* ctx, int32_t op, float* out, const float* in,
                                      int64_t n);

/* ---------------------------------------------------------------- fused loss ------------ */
/* nn.CrossEntropyLoss (nn/loss.mojo:45-61) on logits [B, C] and targets [B, C] as one launch each way.
 *   mtl_cross_entropy_fwd   loss[0] = scale * SUM(y_true * LogSoftmax(logits, axis 1)); equals the nine
 *                           operator calls MAX, SUB, EXP, SUM, LOG, SUB, MUL, SUM, MUL(scale) of the
 *                           reference's graph (same fp32 operations per row; only the final sum over
 *                           rows runs in another order).  The reference's scale is -1 / B.
 *   mtl_cross_entropy_bwd   dlogits (+)= gradient of that loss for an upper gradient of 1: the nine
 *                           backward calls in reverse, MAX.backward's even split among ties included.
 *   mtl_cross_entropy_fwd_grad  both in one launch: the same loss and, overwritten, the same dlogits --
 *                           for a training step, where the backward pass follows the forward with the
 *                           logits and targets unchanged (Model.forward then Model.backward,
 *                           nn/model.mojo:113-330).
 * The intermediate tensors of the nine nodes are not produced.  At most MTL_CROSS_ENTROPY_MAX_ELEMENTS
 * logits per call (the forward is a single block); larger losses go through the operator calls. */
#define MTL_CROSS_ENTROPY_MAX_ELEMENTS (1ll << 22)
MTL_API int32_t mtl_cross_entropy_fwd(mtl_ctx* ctx, float* loss, const float* logits, const float* y_true,
                                      int64_t B, int64_t C, float scale);
MTL_API int32_t mtl_cross_entropy_bwd(mtl_ctx* ctx, float* dlogits, const float* logits, const float* y_true,
                                      int64_t B, int64_t C, float scale, int32_t accumulate);
MTL_API int32_t mtl_cross_entropy_fwd_grad(mtl_ctx* ctx, float* loss, float* dlogits, const float* logits,
                                           const float* y_true, int64_t B, int64_t C, float scale);

/* ---------------------------------------------------------------- optimizer ------------- */

/* Adam.step (mantle/nn/optim.mojo:94-140) over one flat fp32 span of n parameters:
 *   m = b1*m + (1-b1)*g;  v = b2*v + (1-b2)*g*g;
 *   p -= lr * (m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps)
 * with g = grad_scale * grads[i] (grad_scale = 1/world for data-parallel sums). `t` is the
 * 1-based iteration count after the increment at optim.mojo:96. */
MTL_API int32_t mtl_adam_step(mtl_ctx* ctx, float* params, const float* grads, float* m,
                              float* v, int64_t n, float lr, float beta1, float beta2,
                              float eps, int32_t t, float grad_scale);

/* Same step with the iteration count kept in device memory: `t_dev` (one int32, start it at 0)
 * holds the number of steps taken; the update runs as step *t_dev + 1 and stores that number back
 * when it is done, so the call can sit inside a captured step that is replayed many times
 * (Adam.iter, optim.mojo:59,96). */
MTL_API int32_t mtl_adam_step_dev(mtl_ctx* ctx, float* params, const float* grads, float* m,
                                  float* v, int64_t n, float lr, float beta1, float beta2,
                                  float eps, int32_t* t_dev, float grad_scale);

/* ---------------------------------------------------------------- stream capture -------- */

/* Records every call made on the context between begin and end into a CUDA graph; launching it
 * replays a whole training step with one submission.  Shapes in Mantle graphs are compile-time
 * constants (model.mojo:113-171), so a step never changes between replays. */
MTL_API int32_t mtl_graph_begin(mtl_ctx* ctx);
MTL_API int32_t mtl_graph_end(mtl_ctx* ctx, mtl_graph** out);
MTL_API int32_t mtl_graph_launch(mtl_ctx* ctx, mtl_graph* g);
MTL_API int32_t mtl_graph_destroy(mtl_ctx* ctx, mtl_graph* g);

/* ---------------------------------------------------------------- timing ---------------- */

/* CUDA-event stopwatch on the context's stream (replaces the unhooked PerfMetrics table,
 * mantle/autograd/perf_utils.mojo:60-236). slot in [0, 64). */
MTL_API int32_t mtl_timer_start(mtl_ctx* ctx, int32_t slot);
MTL_API int32_t mtl_timer_stop(mtl_ctx* ctx, int32_t slot);
/* Waits for the stop event and returns milliseconds. */
MTL_API int32_t mtl_timer_elapsed_ms(mtl_ctx* ctx, int32_t slot, float* out_ms);

/* Per-kernel device timing of the tensor-core kernels (the dominant launches of a training
 * step): while enabled, and outside stream capture, each launch of the kernel `which` is bracketed
 * by CUDA events on the context's stream.  mtl_prof_get waits for them and returns the summed
 * duration and the launch count since the last reset. */
enum mtl_prof_kernel {
    MTL_PROF_DOT_TC = 0,       /* tcgen05 GEMM behind OP.DOT                          */
    MTL_PROF_CONV_IGEMM = 1,   /* tcgen05 implicit GEMM: CONV2D forward / input grad  */
    MTL_PROF_CONV_WGRAD = 2,   /* tcgen05 implicit GEMM: CONV2D kernel gradient       */
    MTL_PROF_CONV_FIRST = 3,   /* tcgen05 first-layer CONV2D + RELU + MAXPOOL2D       */
    MTL_PROF_KERNELS = 4
};
MTL_API int32_t mtl_prof_enable(mtl_ctx* ctx, int32_t on);
MTL_API int32_t mtl_prof_reset(mtl_ctx* ctx);
MTL_API int32_t mtl_prof_get(mtl_ctx* ctx, int32_t which, float* total_ms, int32_t* launches);

/* Caller-tagged ranges: per-node timing in the manner of PerfMetrics.start_forward_pass /
 * end_forward_pass(pos) (mantle/autograd/perf_utils.mojo:60-112), measured on the device.  While
 * profiling is enabled (mtl_prof_enable) and no capture is in progress, everything enqueued on the
 * context between begin(tag) and end is bracketed by CUDA events; ranges do not nest.  A caller
 * that runs a graph tags each node with its index.  mtl_prof_range_get waits for range i and
 * returns its tag, duration and the number of kernels launched inside it; mtl_prof_dump writes one
 * CSV line per tag (ranges, kernel launches, total / mean milliseconds, share) followed by the
 * per-kernel totals of mtl_prof_get.  mtl_prof_reset clears ranges too. */
MTL_API int32_t mtl_prof_range_begin(mtl_ctx* ctx, int32_t tag);
MTL_API int32_t mtl_prof_range_end(mtl_ctx* ctx);
MTL_API int32_t mtl_prof_range_count(mtl_ctx* ctx, int32_t* out_n);
MTL_API int32_t mtl_prof_range_get(mtl_ctx* ctx, int32_t i, int32_t* tag, float* ms, int32_t* launches);
MTL_API int32_t mtl_prof_dump(mtl_ctx* ctx, const char* path);

/* ---------------------------------------------------------------- data parallel --------- */

/* Data-parallel training is new in this backend (the reference is single-process).  One process
 * per GPU; rank 0 obtains an id, the launcher distributes its 128 bytes, every rank joins. */
#define MTL_DP_ID_BYTES 128
MTL_API int32_t mtl_dp_get_unique_id(uint8_t* out_id /* host, MTL_DP_ID_BYTES */);
MTL_API int32_t mtl_dp_init(mtl_ctx* ctx, const uint8_t* id, int32_t rank, int32_t world);
/* Joining waits for every rank, but not for ever: after MANTLE_DP_INIT_TIMEOUT_S seconds (default
 * 120) mtl_dp_init returns MTL_ERR_COMM naming the rank that gave up, so that a rank that is late or
 * never starts cannot hang the others' hosts.
 *   mtl_dp_probe   the same rendezvous without a context, as a launcher's preflight: joins the group
 *                  within timeout_ms and leaves it again; MTL_OK when every rank arrived in time.
 *                  Use a fresh id for it (an id serves one group).
 *   mtl_dp_status  polls the collective library for an asynchronous error (a peer that died, a
 *                  network fault).  On error the communicator is aborted, MTL_ERR_COMM is returned and
 *                  every later mtl_dp_allreduce_async / mtl_dp_broadcast fails fast with the same
 *                  code.  Host-only and cheap: call it between steps, never inside a capture. */
MTL_API int32_t mtl_dp_probe(const uint8_t* id, int32_t rank, int32_t world, int32_t timeout_ms);
MTL_API int32_t mtl_dp_status(mtl_ctx* ctx);
/* Sum-allreduce of `n` floats in place on a communication stream, ordered after everything
 * enqueued on the context's stream so far; overlaps with later launches until mtl_dp_wait. */
MTL_API int32_t mtl_dp_allreduce_async(mtl_ctx* ctx, float* buf, int64_t n);
/* The same sum for the LAST bucket of a step, which has nothing left to overlap with.  When every rank of the
 * group runs on this machine and could map every other rank's exchange buffer (CUDA IPC, decided once in
 * mtl_dp_init; MANTLE_DP_TAIL_EXCHANGE=0 on any rank switches it off for the group) and n is at most 16384,
 * ONE kernel on the context's stream pushes the values into the peers' buffers over NVLink and collects
 * theirs, summing in rank order, so every rank holds the same bits when the kernel ends: no communication
 * stream, no mtl_dp_wait needed for it.  Every rank must call it the same number of times with the same n.  A
 * peer that does not answer within 20 s ends the wait: the kernel writes MTL_ERR_TIMEOUT to the status word
 * (mtl_device_status), leaves `buf` unsummed and returns.  Otherwise the call is mtl_dp_allreduce_async. */
MTL_API int32_t mtl_dp_allreduce_tail(mtl_ctx* ctx, float* buf, int64_t n);
/* 1 when mtl_dp_allreduce_tail exchanges directly, 0 when it falls back to the collective library. */
MTL_API int32_t mtl_dp_tail_exchange_enabled(mtl_ctx* ctx);
/* Self-test of that exchange on ONE GPU: `world` emulated ranks (2..8) in one cooperative launch, rank r
 * owning grads[r*n .. r*n+n) (device memory), `steps` exchanges in a row; afterwards every rank's slice
 * holds the rank-ordered sum.  With silent_rank >= 0 that rank never pushes and the others give up after
 * budget_us microseconds: the status word reads MTL_ERR_TIMEOUT and their slices are unchanged. */
MTL_API int32_t mtl_selftest_tail_exchange(mtl_ctx* ctx, float* grads, int32_t world, int32_t n, int32_t steps,
                                           int32_t silent_rank, int32_t budget_us);
/* Makes the context's stream wait for all outstanding allreduces. */
MTL_API int32_t mtl_dp_wait(mtl_ctx* ctx);
/* Host callback of the fused CONV2D backward entry points (mtl_conv2d_bwd_fused*, mtl_conv2d_bwd_pooled):
 * when they compute dX as well, `hook(user)` is called once every kernel that writes dW and db has been
 * enqueued and before the kernels of dX, so that a data-parallel caller can start exchanging the
 * layer's parameter gradients (mtl_dp_allreduce_async) while the input gradient is computed.  Paths
 * that cannot separate the two do not call it; the caller learns from its own flag whether it ran.
 * Pass a null hook to remove it. */
MTL_API int32_t mtl_set_grads_ready_hook(mtl_ctx* ctx, void (*hook)(void* user), void* user);
/* Broadcast `n` floats from `root` (initial parameters). */
MTL_API int32_t mtl_dp_broadcast(mtl_ctx* ctx, float* buf, int64_t n, int32_t root);
MTL_API int32_t mtl_dp_destroy(mtl_ctx* ctx);
/* Number of ranks joined by mtl_dp_init, 1 when the context is not part of a group. */
MTL_API int32_t mtl_dp_world_size(mtl_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* MANTLE_CUDA_H_ */
