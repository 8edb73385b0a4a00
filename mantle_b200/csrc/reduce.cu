// SUM / MEAN / MAX forward and backward.  Whole-tensor reductions run as a deterministic two-pass
// tree (per-block partials in scratch, then one block), axis reductions as one thread or one block
// per output element depending on the axis length.  Warp-shuffle reductions throughout.
#include <float.h>

#include "common.cuh"

namespace {

constexpr int kBlock = 256;

enum { R_SUM = 0, R_MAX = 1, R_COUNT_EQ = 2 };

template <int MODE>
__device__ __forceinline__ float r_init() { return MODE == R_MAX ? -FLT_MAX : 0.0f; }
template <int MODE>
__device__ __forceinline__ float r_comb(float a, float b) { return MODE == R_MAX ? fmaxf(a, b) : a + b; }
template <int MODE>
__device__ __forceinline__ float r_load(float x, float ref) {
    return MODE == R_COUNT_EQ ? (x == ref ? 1.0f : 0.0f) : x;
}

template <int MODE>
__device__ __forceinline__ float block_reduce(float v, float* smem) {
    const int COMB = MODE == R_MAX ? R_MAX : R_SUM;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = r_comb<COMB>(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = r_init<COMB>();
    if (threadIdx.x < 32) {
        t = threadIdx.x < (blockDim.x >> 5) ? smem[threadIdx.x] : r_init<COMB>();
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t = r_comb<COMB>(t, __shfl_xor_sync(0xffffffffu, t, o));
    }
    __syncthreads();
    return t;  // valid in thread 0
}

// pass 1: each block reduces a grid-strided slice of `in` to partial[blockIdx.x]
template <int MODE>
__global__ void __launch_bounds__(kBlock) k_reduce_partial(float* __restrict__ partial, const float* __restrict__ in,
                                                           int64_t n, const float* __restrict__ ref) {
    __shared__ float smem[32];
    const int COMB = MODE == R_MAX ? R_MAX : R_SUM;
    float rv = MODE == R_COUNT_EQ ? __ldg(ref) : 0.0f;
    float acc = r_init<COMB>();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if ((((uintptr_t)in) & 15u) == 0) {
        int64_t n4 = n >> 2;
        const float4* in4 = reinterpret_cast<const float4*>(in);
        for (int64_t i = tid; i < n4; i += stride) {
            float4 v = in4[i];
            acc = r_comb<COMB>(acc, r_load<MODE>(v.x, rv));
            acc = r_comb<COMB>(acc, r_load<MODE>(v.y, rv));
            acc = r_comb<COMB>(acc, r_load<MODE>(v.z, rv));
            acc = r_comb<COMB>(acc, r_load<MODE>(v.w, rv));
        }
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride) acc = r_comb<COMB>(acc, r_load<MODE>(in[i], rv));
    } else {
        for (int64_t i = tid; i < n; i += stride) acc = r_comb<COMB>(acc, r_load<MODE>(in[i], rv));
    }
    float t = block_reduce<MODE>(acc, smem);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

// pass 2: one block folds the partials; out = result * scale
template <int MODE>
__global__ void __launch_bounds__(kBlock) k_reduce_final(float* __restrict__ out, const float* __restrict__ partial,
                                                         int n_partial, float scale, int divide) {
    __shared__ float smem[32];
    const int COMB = MODE == R_MAX ? R_MAX : R_SUM;
    float acc = r_init<COMB>();
    for (int i = threadIdx.x; i < n_partial; i += blockDim.x) acc = r_comb<COMB>(acc, partial[i]);
    float t = block_reduce<COMB>(acc, smem);
    if (threadIdx.x == 0) out[0] = divide ? t / scale : t;
}

// POW.backward for the exponent, pass 1: partial[block] = sum over a grid-strided slice of
// x^a * log(x) * ug, with log(x) taken as 0 where it is infinite (x == 0), basics.mojo:359-376.
__global__ void __launch_bounds__(kBlock) k_pow_exponent_partial(float* __restrict__ partial, const float* __restrict__ x,
                                                                 const float* __restrict__ ug, int64_t n, float a) {
    __shared__ float smem[32];
    float acc = 0.0f;
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) {
        const float v = x[i];
        float lg = logf(v);
        if (isinf(lg)) lg = 0.0f;
        acc += powf(v, a) * lg * ug[i];
    }
    float t = block_reduce<R_SUM>(acc, smem);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
}

// pass 2: one block folds the partials into the [1]-shaped gradient
__global__ void __launch_bounds__(kBlock) k_pow_exponent_final(float* __restrict__ grad, const float* __restrict__ partial,
                                                               int n_partial, int acc) {
    __shared__ float smem[32];
    float v = 0.0f;
    for (int i = threadIdx.x; i < n_partial; i += blockDim.x) v += partial[i];
    float t = block_reduce<R_SUM>(v, smem);
    if (threadIdx.x == 0) grad[0] = acc ? grad[0] + t : t;
}

// Axis reduction, one thread per output element (short axes).
template <int MODE>
__global__ void __launch_bounds__(kBlock) k_reduce_axis_thread(float* __restrict__ out, const float* __restrict__ in,
                                                               int64_t n_out, int64_t stride_ax, int64_t dim,
                                                               int mean) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t gstride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n_out; i += gstride) {
        // index_base of reduce (tensorutils.mojo:655-657)
        int64_t base = (i % stride_ax) + (i / stride_ax) * (stride_ax * dim);
        float acc = r_init<MODE>();
        for (int64_t j = 0; j < dim; ++j) acc = r_comb<MODE>(acc, in[base + j * stride_ax]);
        out[i] = mean ? acc / (float)dim : acc;
    }
}

// Axis reduction, one block per output element (long axes).
template <int MODE>
__global__ void __launch_bounds__(kBlock) k_reduce_axis_block(float* __restrict__ out, const float* __restrict__ in,
                                                              int64_t n_out, int64_t stride_ax, int64_t dim,
                                                              int mean) {
    __shared__ float smem[32];
    for (int64_t i = blockIdx.x; i < n_out; i += gridDim.x) {
        int64_t base = (i % stride_ax) + (i / stride_ax) * (stride_ax * dim);
        float acc = r_init<MODE>();
        for (int64_t j = threadIdx.x; j < dim; j += blockDim.x) acc = r_comb<MODE>(acc, in[base + j * stride_ax]);
        float t = block_reduce<MODE>(acc, smem);
        if (threadIdx.x == 0) out[i] = mean ? t / (float)dim : t;
    }
}

// SUM / MEAN backward along an axis, and the whole-tensor forms: grad[i] (+)= coef * ug[u(i)].
// `twice` reproduces accumulate_op applying its function twice when both shapes are equal
// (tensorutils.mojo:380-393): the factor ug enters squared.
__global__ void __launch_bounds__(kBlock) k_sum_mean_bwd(float* __restrict__ grad, const float* __restrict__ ug,
                                                         int64_t n, int64_t stride_ax, int64_t dim, int all,
                                                         float coef, int twice, int acc) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t gstride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += gstride) {
        int64_t u = all ? 0 : (i % stride_ax) + (i / (stride_ax * dim)) * stride_ax;
        float g = ug[u];
        float r = coef * g;
        if (twice) r = r * g;
        grad[i] = acc ? grad[i] + r : r;
    }
}

// MAX backward, whole tensor: stats[0] = max, stats[1] = number of elements equal to it.
__global__ void __launch_bounds__(kBlock) k_max_bwd_all(float* __restrict__ grad, const float* __restrict__ ug,
                                                        const float* __restrict__ in, const float* __restrict__ stats,
                                                        int64_t n, int acc) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t gstride = (int64_t)gridDim.x * blockDim.x;
    float mx = stats[0];
    float factor = 1.0f / stats[1];
    float g = factor * ug[0];
    for (int64_t i = tid; i < n; i += gstride) {
        float r = in[i] == mx ? g : 0.0f;
        grad[i] = acc ? grad[i] + r : r;
    }
}

// MAX backward along an axis: one thread per reduced row (basics.mojo:597-613).
__global__ void __launch_bounds__(kBlock) k_max_bwd_axis(float* __restrict__ grad, const float* __restrict__ ug,
                                                         const float* __restrict__ in, int64_t n_out,
                                                         int64_t stride_ax, int64_t dim, int acc) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t gstride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n_out; i += gstride) {
        int64_t base = (i % stride_ax) + (i / stride_ax) * (stride_ax * dim);
        float mx = -FLT_MAX;
        for (int64_t j = 0; j < dim; ++j) mx = fmaxf(mx, in[base + j * stride_ax]);
        float cnt = 0.0f;
        for (int64_t j = 0; j < dim; ++j) cnt += in[base + j * stride_ax] == mx ? 1.0f : 0.0f;
        float g = (1.0f / cnt) * ug[i];
        for (int64_t j = 0; j < dim; ++j) {
            int64_t idx = base + j * stride_ax;
            float r = in[idx] == mx ? g : 0.0f;
            grad[idx] = acc ? grad[idx] + r : r;
        }
    }
}

template <int MODE>
int32_t reduce_all(mtl_ctx* ctx, float* out, const float* in, int64_t n, const float* ref, float scale,
                   int divide, float* partial) {
    int blocks = mtl_grid_for((n + 3) / 4, kBlock, ctx->sm_count, 4);
    k_reduce_partial<MODE><<<blocks, kBlock, 0, ctx->stream>>>(partial, in, n, ref);
    MTL_LAUNCHED(ctx);
    k_reduce_final<MODE><<<1, kBlock, 0, ctx->stream>>>(out, partial, blocks, scale, divide);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

bool reduce_args_ok(int32_t rank, const int64_t* shape, int32_t axis) {
    if (rank < 1 || rank > MTL_MAX_RANK || !shape) return false;
    for (int i = 0; i < rank; ++i)
        if (shape[i] < 1) return false;
    return axis < rank;
}

}  // namespace

extern "C" {

int32_t mtl_reduce_fwd(mtl_ctx* ctx, int32_t op, float* out, const float* in, int32_t rank,
                       const int64_t* shape, int32_t axis) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, op == MTL_OP_SUM || op == MTL_OP_MEAN || op == MTL_OP_MAX,
                "mtl_reduce_fwd: op id %d is not SUM/MEAN/MAX", op);
    MTL_REQUIRE(ctx, out && in && reduce_args_ok(rank, shape, axis), "bad arguments to mtl_reduce_fwd");
    int64_t n = mtl_numel(rank, shape);
    if (axis < 0) {
        void* ws;
        int32_t rc = mtl_workspace(ctx, 4096 * sizeof(float), &ws);
        if (rc) return rc;
        float* partial = (float*)ws;
        if (op == MTL_OP_MAX) return reduce_all<R_MAX>(ctx, out, in, n, nullptr, 1.0f, 0, partial);
        return reduce_all<R_SUM>(ctx, out, in, n, nullptr, (float)n, op == MTL_OP_MEAN, partial);
    }
    int64_t dim = shape[axis];
    int64_t stride_ax = 1;
    for (int d = axis + 1; d < rank; ++d) stride_ax *= shape[d];
    int64_t n_out = n / dim;
    int mean = op == MTL_OP_MEAN;
    if (dim >= 512) {
        int grid = (int)(n_out < (int64_t)ctx->sm_count * 8 ? n_out : (int64_t)ctx->sm_count * 8);
        if (op == MTL_OP_MAX)
            k_reduce_axis_block<R_MAX><<<grid, kBlock, 0, ctx->stream>>>(out, in, n_out, stride_ax, dim, 0);
        else
            k_reduce_axis_block<R_SUM><<<grid, kBlock, 0, ctx->stream>>>(out, in, n_out, stride_ax, dim, mean);
    } else {
        int grid = mtl_grid_for(n_out, kBlock, ctx->sm_count, 8);
        if (op == MTL_OP_MAX)
            k_reduce_axis_thread<R_MAX><<<grid, kBlock, 0, ctx->stream>>>(out, in, n_out, stride_ax, dim, 0);
        else
            k_reduce_axis_thread<R_SUM><<<grid, kBlock, 0, ctx->stream>>>(out, in, n_out, stride_ax, dim, mean);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_reduce_bwd(mtl_ctx* ctx, int32_t op, float* grad, const float* ug, const float* in,
                       int32_t rank, const int64_t* shape, int32_t axis, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, op == MTL_OP_SUM || op == MTL_OP_MEAN || op == MTL_OP_MAX,
                "mtl_reduce_bwd: op id %d is not SUM/MEAN/MAX", op);
    MTL_REQUIRE(ctx, grad && ug && reduce_args_ok(rank, shape, axis), "bad arguments to mtl_reduce_bwd");
    MTL_REQUIRE(ctx, op != MTL_OP_MAX || in, "MAX backward needs the forward input");
    int64_t n = mtl_numel(rank, shape);
    int acc = accumulate ? 1 : 0;
    int64_t dim = axis >= 0 ? shape[axis] : n;
    int64_t stride_ax = 1;
    for (int d = axis + 1; axis >= 0 && d < rank; ++d) stride_ax *= shape[d];
    int grid = mtl_grid_for(n, kBlock, ctx->sm_count, 8);

    if (op == MTL_OP_SUM || op == MTL_OP_MEAN) {
        float coef = 1.0f;
        int twice = 0;
        if (op == MTL_OP_SUM) {
            // SUM.backward: fill(1) then accumulate_op[mul] with ug (basics.mojo:416-425)
            twice = (axis >= 0) ? (dim == 1) : (rank == 1 && shape[0] == 1);
        } else if (axis < 0) {
            coef = (float)(1.0 / (double)n);  // basics.mojo:477-483
        } else {
            coef = (float)(1.0 / (double)dim);  // basics.mojo:500-504
            twice = dim == 1;
        }
        k_sum_mean_bwd<<<grid, kBlock, 0, ctx->stream>>>(grad, ug, n, stride_ax, dim, axis < 0, coef, twice, acc);
        MTL_LAUNCHED(ctx);
        return MTL_OK;
    }
    if (axis < 0) {
        void* ws;
        int32_t rc = mtl_workspace(ctx, 8192 * sizeof(float), &ws);
        if (rc) return rc;
        float* stats = (float*)ws;        // [0] max, [1] tie count
        float* partial = stats + 64;
        rc = reduce_all<R_MAX>(ctx, stats, in, n, nullptr, 1.0f, 0, partial);
        if (rc) return rc;
        rc = reduce_all<R_COUNT_EQ>(ctx, stats + 1, in, n, stats, 1.0f, 0, partial);
        if (rc) return rc;
        k_max_bwd_all<<<grid, kBlock, 0, ctx->stream>>>(grad, ug, in, stats, n, acc);
        MTL_LAUNCHED(ctx);
        return MTL_OK;
    }
    int64_t n_out = n / dim;
    int g2 = mtl_grid_for(n_out, kBlock, ctx->sm_count, 8);
    k_max_bwd_axis<<<g2, kBlock, 0, ctx->stream>>>(grad, ug, in, n_out, stride_ax, dim, acc);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_pow_bwd_exponent(mtl_ctx* ctx, float* grad, const float* ug, const float* in, int64_t n, float exponent,
                             int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, grad && ug && in && n >= 1, "bad arguments to mtl_pow_bwd_exponent");
    int blocks = mtl_grid_for(n, kBlock, ctx->sm_count, 4);
    if (blocks > 1024) blocks = 1024;
    void* ws;
    int32_t rc = mtl_workspace(ctx, 1024 * sizeof(float), &ws);
    if (rc) return rc;
    k_pow_exponent_partial<<<blocks, kBlock, 0, ctx->stream>>>((float*)ws, in, ug, n, exponent);
    MTL_LAUNCHED(ctx);
    k_pow_exponent_final<<<1, kBlock, 0, ctx->stream>>>(grad, (const float*)ws, blocks, accumulate ? 1 : 0);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

// ------------------------------------------------------------------ no-allocation variant ----
// Scratch for mtl_reduce_all_static: one partial per block of the first pass.  It lives in the
// library image, so every GPU that loads the library carries these 4 KB until the process exits.
#define MTL_STATIC_REDUCE_BLOCKS 1024
static __device__ __align__(256) float g_static_reduce_partials[MTL_STATIC_REDUCE_BLOCKS];

// Device address of the array above for each device ordinal, resolved on first use.  In host code
// the array's name only stands for the symbol; a kernel must be handed the address that
// cudaGetSymbolAddress reports for the device that is current.  The cache is written without a
// lock: two host threads that race on a device's first call both store the same address.
static float* g_static_reduce_addr[64] = {nullptr};

int32_t mtl_reduce_all_static(mtl_ctx* ctx, int32_t op, float* out, const float* in, int64_t n) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, op == MTL_OP_SUM || op == MTL_OP_MEAN || op == MTL_OP_MAX,
                "mtl_reduce_all_static: op id %d is not SUM/MEAN/MAX", op);
    MTL_REQUIRE(ctx, out && in, "null pointer in mtl_reduce_all_static");
    MTL_REQUIRE(ctx, n >= 1 && n <= MTL_REDUCE_STATIC_MAX_ELEMENTS,
                "mtl_reduce_all_static handles 1..%lld elements, got %lld; use mtl_reduce_fwd for larger tensors",
                (long long)MTL_REDUCE_STATIC_MAX_ELEMENTS, (long long)n);
    MTL_REQUIRE(ctx, ctx->device >= 0 && ctx->device < 64, "device ordinal %d out of range", ctx->device);
    float* partial = g_static_reduce_addr[ctx->device];
    if (!partial) {
        // one-time set-up for this device (it is current here: every entry point makes its context's
        // device current and restores the caller's on return): ask where the array lives on it.
        // The lookup may load the module, which must not happen inside a stream capture.
        MTL_REQUIRE(ctx, !ctx->capturing,
                    "the first mtl_reduce_all_static call on a device must come before stream capture starts");
        void* p = nullptr;
        MTL_CUDA(ctx, cudaGetSymbolAddress(&p, g_static_reduce_partials));
        partial = g_static_reduce_addr[ctx->device] = (float*)p;
    }
    int blocks = mtl_grid_for((n + 3) / 4, kBlock, ctx->sm_count, 4);
    if (blocks > MTL_STATIC_REDUCE_BLOCKS) blocks = MTL_STATIC_REDUCE_BLOCKS;
    // every partial[0..blocks) is written by the first pass before the second reads it, so nothing
    // left over from an earlier call has to be cleared
    if (op == MTL_OP_MAX) {
        k_reduce_partial<R_MAX><<<blocks, kBlock, 0, ctx->stream>>>(partial, in, n, nullptr);
        MTL_LAUNCHED(ctx);
        k_reduce_final<R_MAX><<<1, kBlock, 0, ctx->stream>>>(out, partial, blocks, 1.0f, 0);
    } else {
        k_reduce_partial<R_SUM><<<blocks, kBlock, 0, ctx->stream>>>(partial, in, n, nullptr);
        MTL_LAUNCHED(ctx);
        k_reduce_final<R_SUM><<<1, kBlock, 0, ctx->stream>>>(out, partial, blocks, (float)n, op == MTL_OP_MEAN);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

}  // extern "C"
