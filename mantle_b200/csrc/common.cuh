// Internal declarations shared by the translation units of libmantle_cuda.so.
#pragma once

#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <string>
#include <utility>
#include <vector>

#include "../../include/mantle_cuda.h"

#define MTL_NUM_TIMERS 64

// Tuning switches, read from the environment ONCE when a context is created (the launch paths never
// call getenv).  A negative value means "not set: use the built-in choice".
struct mtl_tuning {
    bool log_errors = false;          // MANTLE_CUDA_LOG=1: print every recorded error to stderr
    bool conv_channel_major = true;   // MANTLE_CONV_CHANNEL_MAJOR=0 switches the channel-major implicit GEMM off
    bool conv_paired = true;          // MANTLE_CONV_PAIRED=0: one filter tap per instruction
    int conv_tail_split = 0;           // MANTLE_CONV_TAIL_SPLIT=0: tiles of a partial last wave are never split along k
    int conv_paired_min_kblocks = 32;  // MANTLE_CONV_PAIRED_MIN_KB: shortest reduction (k-blocks per tile) that pairs taps
    bool conv_spread = true;          // MANTLE_CONV_SPREAD=0: plain row order of the pixel boxes
    bool conv_pool_epilogue = true;   // MANTLE_CONV_POOL_EPILOGUE=0: conv -> ReLU -> pool through scratch memory
    bool conv_first_tc = true;        // MANTLE_CONV_FIRST_TC=0: first layer on the CUDA-core kernels in every mode
    bool gemm_3d_boxes = true;        // MANTLE_GEMM_NO3D set: one 2-D box per 32-wide chunk of an MN-major operand
    int wgrad_taps = -1;              // MANTLE_WGRAD_TAPS: filter taps per CTA of the kernel gradient
    int gemm_bn = -1;                 // MANTLE_GEMM_BN: DOT tile width (128 / 256)
    int gemm_mt = -1;                 // MANTLE_GEMM_MT: 1 = 128-row tiles, 2 = 256-row tiles
    int gemm_stages = -1;             // MANTLE_GEMM_STAGES: operand ring depth
    int gemm_split_k = -1;            // MANTLE_GEMM_SPLITK=1: stream-K schedule for DOT when whole tiles leave SMs idle
    bool pdl = true;                  // MANTLE_PDL=0: plain stream order between the kernels of a step
    bool debug_guards = false;        // MANTLE_CUDA_DEBUG=1: guard words around every mtl_malloc block, checked at mtl_sync
};

struct mtl_ctx {
    int device = 0;
    mtl_tuning tune;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int math_mode = MTL_MATH_TF32X3;
    int sm_count = 148;        // SMs the persistent grids may use (a data-parallel group takes some off)
    int sm_count_total = 148;  // SMs of the device
    // scratch workspace, grown on demand outside capture
    void* ws = nullptr;
    size_t ws_bytes = 0;
    void* ws2 = nullptr;  // second scratch block (mtl_workspace2)
    size_t ws2_bytes = 0;
    int64_t conv_split_tiles = 0;   // mtl_conv_split_tiles
    void* split_scratch = nullptr;  // partial accumulators of k-split tail tiles (mtl_split_scratch), fixed size
    bool capturing = false;
    // Instantiated graphs of this context that are alive.  They hold the scratch pointers that were
    // current when they were captured, so while any is alive a scratch block that has to grow is not
    // freed but parked on `retired` (freed when the last graph goes, or with the context).
    int live_graphs = 0;
    std::vector<void*> retired;
    // debug guards (tune.debug_guards): user pointer -> payload bytes of every live mtl_malloc block
    std::vector<std::pair<void*, size_t>> guarded;
    int64_t launches = 0;
    int64_t launches_at_capture = 0;
    int32_t* dev_status = nullptr;  // one word written by bounded device waits
    // 8192 zeroed counters behind the status word: kernels that fold their own partial results count
    // the blocks that have finished a group here; the block that folds puts the counter back to zero
    int32_t* tickets = nullptr;
    char err[512] = {0};
    cudaEvent_t t0[MTL_NUM_TIMERS] = {0};
    cudaEvent_t t1[MTL_NUM_TIMERS] = {0};
    // data parallel state (dp.cu)
    void* dp = nullptr;
    // cached driver entry point for tensor-map encoding (tma.cuh)
    void* encode_tiled = nullptr;
    void (*grads_ready_hook)(void*) = nullptr;  // see mtl_set_grads_ready_hook
    void* grads_ready_user = nullptr;
    // staged input copies (mtl_stage_*): a copy stream and two events per slot
    cudaStream_t copy_stream = nullptr;
    cudaEvent_t stage_ready[4] = {0};
    cudaEvent_t stage_free[4] = {0};
    bool stage_released[4] = {false, false, false, false};
    // per-kernel event timing (mtl_prof_*)
    bool prof_on = false;
    std::vector<std::pair<cudaEvent_t, cudaEvent_t>> prof_events[MTL_PROF_KERNELS];
    // caller-tagged ranges (mtl_prof_range_*): everything enqueued between begin and end
    struct prof_range { int32_t tag; cudaEvent_t e0, e1; int64_t launches; };
    std::vector<prof_range> ranges;
    bool range_open = false;
    prof_range open_range = {0, nullptr, nullptr, 0};
};

// Brackets one launch of a profiled kernel with events when profiling is on.
struct mtl_prof_scope {
    mtl_ctx* ctx;
    int which;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    mtl_prof_scope(mtl_ctx* c, int w) : ctx(c), which(w) {
        if (ctx->prof_on && !ctx->capturing && cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess)
            cudaEventRecord(e0, ctx->stream);
        else
            e0 = e1 = nullptr;
    }
    ~mtl_prof_scope() {
        if (e0 && e1) {
            cudaEventRecord(e1, ctx->stream);
            ctx->prof_events[which].push_back({e0, e1});
        }
    }
};

struct mtl_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    int64_t launches = 0;  // kernels recorded in the graph
};

int32_t mtl_set_error(mtl_ctx* ctx, int32_t code, const char* fmt, ...);
// The environment switches, read once per process on first use (contexts copy them at creation).
const mtl_tuning& mtl_global_tuning();
// Returns a device pointer to at least `bytes` of scratch, 256-byte aligned.
int32_t mtl_workspace(mtl_ctx* ctx, size_t bytes, void** out);
int32_t mtl_workspace2(mtl_ctx* ctx, size_t bytes, void** out);
int32_t mtl_split_scratch(mtl_ctx* ctx, void** out);

// Makes the context's device current for the duration of an entry point and puts the caller's
// device back afterwards, so that one host thread can drive contexts on different GPUs in turn.
struct mtl_device_guard {
    int prev = -1;
    bool switched = false;
    explicit mtl_device_guard(int device) {
        if (cudaGetDevice(&prev) != cudaSuccess) { cudaGetLastError(); prev = -1; }
        if (prev != device) switched = cudaSetDevice(device) == cudaSuccess;
    }
    ~mtl_device_guard() {
        if (switched && prev >= 0) cudaSetDevice(prev);
    }
    mtl_device_guard(const mtl_device_guard&) = delete;
    mtl_device_guard& operator=(const mtl_device_guard&) = delete;
};

// First statement of every entry point that takes a context: rejects a null context and makes the
// context's device current until the entry point returns.
#define MTL_CHECK_CTX(ctx)                  \
    if (!(ctx)) return MTL_ERR_INVALID;     \
    mtl_device_guard mtl_guard__((ctx)->device)

#define MTL_REQUIRE(ctx, cond, ...)                                  \
    do {                                                             \
        if (!(cond)) return mtl_set_error(ctx, MTL_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define MTL_CUDA(ctx, call)                                                              \
    do {                                                                                 \
        cudaError_t e__ = (call);                                                        \
        if (e__ != cudaSuccess)                                                          \
            return mtl_set_error(ctx, MTL_ERR_CUDA, "%s failed: %s (%s:%d)", #call,      \
                                 cudaGetErrorString(e__), __FILE__, __LINE__);           \
    } while (0)

// After a kernel launch: count it and surface launch-configuration errors.
#define MTL_LAUNCHED(ctx)                                                                \
    do {                                                                                 \
        (ctx)->launches++;                                                               \
        cudaError_t e__ = cudaPeekAtLastError();                                         \
        if (e__ != cudaSuccess) {                                                        \
            cudaGetLastError();                                                          \
            return mtl_set_error(ctx, MTL_ERR_CUDA, "kernel launch failed: %s (%s:%d)",  \
                                 cudaGetErrorString(e__), __FILE__, __LINE__);           \
        }                                                                                \
    } while (0)

// ---- programmatic dependent launch ---------------------------------------------------------
// A training step at small batches is a chain of short kernels, and the gap between two of them
// (the first one draining, the second one being scheduled and setting itself up) is paid two dozen
// times per step.  Kernels launched through mtl_launch_pdl may be scheduled while their predecessor
// in the stream is still running; each of them calls mtl_pdl_sync() before it touches global
// memory, which (1) waits until the predecessor has completed and its writes are visible and
// (2) lets the successor be scheduled in turn.  What overlaps is therefore only a kernel's set-up
// (barrier initialisation, tensor-memory allocation, index arithmetic) and the scheduling itself;
// the order of all memory effects is the stream order, also inside a captured graph.
// EVERY kernel launched this way must call mtl_pdl_sync() before its first global access.
#ifdef __CUDACC__
__device__ __forceinline__ void mtl_pdl_sync() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... Params, typename... Args>
inline void mtl_launch_pdl(mtl_ctx* ctx, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->tune.pdl ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);  // errors surface through MTL_LAUNCHED
}
#endif

static inline int64_t mtl_numel(int32_t rank, const int64_t* shape) {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= shape[i];
    return n;
}

static inline int mtl_grid_for(int64_t work_items, int block, int sm_count, int ctas_per_sm) {
    int64_t g = (work_items + block - 1) / block;
    int64_t cap = (int64_t)sm_count * ctas_per_sm;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (int)g;
}

// ---- entry points implemented across translation units (internal linkage names) ----------
int32_t mtl_gemm_simt(mtl_ctx* ctx, float* C, const float* A, const float* B, int64_t M,
                      int64_t N, int64_t K, int transA, int transB, int accumulate);
// Returns MTL_ERR_UNSUPPORTED when the shape cannot run on the tensor-core kernel.
int32_t mtl_gemm_tc(mtl_ctx* ctx, float* C, const float* A, const float* B, int64_t M,
                    int64_t N, int64_t K, int transA, int transB, int accumulate, int x3);
// Thin products (N <= 16) bound by reading A; re-associates the k sum.
bool mtl_gemm_thin_supported(int64_t M, int64_t N, int64_t K, int transA, int transB);
int32_t mtl_gemm_thin(mtl_ctx* ctx, float* C, const float* A, const float* B, int64_t M, int64_t N, int64_t K,
                      int transA, int accumulate);
bool mtl_gemm_tc_supported(int64_t M, int64_t N, int64_t K, int transA, int transB,
                           const float* A, const float* B, const float* C);
