// Elementwise, broadcast and un-broadcast kernels: fill / copy, the unary op family, the
// ADD/SUB/MUL/DIV family with NumPy broadcasting, FMA.  All are HBM-bound: 128-bit accesses on the
// contiguous paths, grids sized to the SM count with grid-stride loops.
#include "common.cuh"

namespace {

constexpr int kBlock = 256;
constexpr int kCtasPerSm = 8;

__device__ __forceinline__ float powi(float x, int n) {
    // integer power by squaring, the result of Mojo's pow(SIMD, Int) used by elwise_pow
    bool neg = n < 0;
    unsigned e = neg ? (unsigned)(-(long long)n) : (unsigned)n;
    float r = 1.0f, b = x;
    while (e) {
        if (e & 1u) r *= b;
        b *= b;
        e >>= 1;
    }
    return neg ? 1.0f / r : r;
}

struct UnaryFwd {
    int op;
    float p0, p1;
    __device__ __forceinline__ float operator()(float x) const {
        switch (op) {
            case MTL_OP_EXP: return expf(x);
            case MTL_OP_LOG: return logf(x);
            case MTL_OP_POW: return powi(x, (int)p0);
            case MTL_OP_SIGMOID: return 1.0f / (1.0f + expf(-x));
            case MTL_OP_RELU: return x > 0.0f ? x : 0.0f;
            case MTL_OP_TANH: {
                float ep = expf(x), en = expf(-x);
                return (ep - en) / (ep + en);
            }
            case MTL_OP_CLIP: return fmaxf(fminf(x, p1), p0);
            case MTL_OP_LEAKYRELU: return x > 0.0f ? x : x * p0;
            default: return x;
        }
    }
};

struct UnaryBwd {
    int op;
    float p0, p1;
    __device__ __forceinline__ float operator()(float x, float ug) const {
        switch (op) {
            case MTL_OP_EXP: return expf(x) * ug;
            case MTL_OP_LOG: return ug / x;
            case MTL_OP_POW: return p0 * powf(x + 1e-12f, p0 - 1.0f) * ug;
            case MTL_OP_SIGMOID: {
                float s = 1.0f / (1.0f + expf(-x));
                return s * (1.0f - s) * ug;
            }
            case MTL_OP_RELU: return (x > 0.0f ? 1.0f : 0.0f) * ug;
            case MTL_OP_TANH: {
                float ep = expf(x), en = expf(-x);
                float t = (ep - en) / (ep + en);
                return (1.0f - t * t) * ug;
            }
            case MTL_OP_CLIP: return (x >= p0 && x <= p1) ? ug : 0.0f;
            case MTL_OP_LEAKYRELU: return (x > 0.0f ? 1.0f : p0) * ug;
            default: return ug;
        }
    }
};

__device__ __forceinline__ float bin_apply(int op, float a, float b) {
    switch (op) {
        case MTL_OP_ADD: return a + b;
        case MTL_OP_SUB: return a - b;
        case MTL_OP_MUL: return a * b;
        default: return a / b;
    }
}

// out[i] = f(in[i]); float4 body when all pointers are 16-byte aligned.
template <class F>
__global__ void __launch_bounds__(kBlock) k_map1(float* __restrict__ out, const float* __restrict__ in,
                                                 int64_t n, F f, int vec) {
    mtl_pdl_sync();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t n4 = n >> 2;
        const float4* in4 = reinterpret_cast<const float4*>(in);
        float4* out4 = reinterpret_cast<float4*>(out);
        for (int64_t i = tid; i < n4; i += stride) {
            float4 v = in4[i];
            v.x = f(v.x); v.y = f(v.y); v.z = f(v.z); v.w = f(v.w);
            out4[i] = v;
        }
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride) out[i] = f(in[i]);
    } else {
        for (int64_t i = tid; i < n; i += stride) out[i] = f(in[i]);
    }
}

// out[i] (+)= f(x[i], y[i])
template <class F>
__global__ void __launch_bounds__(kBlock) k_map2(float* __restrict__ out, const float* __restrict__ x,
                                                 const float* __restrict__ y, int64_t n, F f, int vec,
                                                 int acc) {
    mtl_pdl_sync();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t n4 = n >> 2;
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const float4* y4 = reinterpret_cast<const float4*>(y);
        float4* out4 = reinterpret_cast<float4*>(out);
        for (int64_t i = tid; i < n4; i += stride) {
            float4 a = x4[i], b = y4[i], r;
            r.x = f(a.x, b.x); r.y = f(a.y, b.y); r.z = f(a.z, b.z); r.w = f(a.w, b.w);
            if (acc) {
                float4 o = out4[i];
                r.x += o.x; r.y += o.y; r.z += o.z; r.w += o.w;
            }
            out4[i] = r;
        }
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride) {
            float r = f(x[i], y[i]);
            out[i] = acc ? out[i] + r : r;
        }
    } else {
        for (int64_t i = tid; i < n; i += stride) {
            float r = f(x[i], y[i]);
            out[i] = acc ? out[i] + r : r;
        }
    }
}

__global__ void __launch_bounds__(kBlock) k_fill(float* __restrict__ p, int64_t n, float v, int vec) {
    mtl_pdl_sync();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t n4 = n >> 2;
        float4 v4 = make_float4(v, v, v, v);
        float4* p4 = reinterpret_cast<float4*>(p);
        for (int64_t i = tid; i < n4; i += stride) p4[i] = v4;
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride) p[i] = v;
    } else {
        for (int64_t i = tid; i < n; i += stride) p[i] = v;
    }
}

struct BinF {
    int op;
    __device__ __forceinline__ float operator()(float x, float y) const { return bin_apply(op, x, y); }
};

struct AddTo {
    __device__ __forceinline__ float operator()(float dst, float src) const { return dst + src; }
};

// Broadcast index space: `shape` is the broadcast (output) shape, sa/sb the operand strides with 0
// on broadcast axes (broadcast_calculate_strides, tensorutils.mojo:150-175).
struct Bcast {
    int rank;
    int narrow;  // all extents and strides fit 32 bits
    int64_t shape[MTL_MAX_RANK];
    int64_t sa[MTL_MAX_RANK];
    int64_t sb[MTL_MAX_RANK];
};

// `narrow` (every extent and offset below 2^31): the same arithmetic in 32 bits, whose divisions
// are several times cheaper; the small tensors of a loss function are bound by exactly these.
__device__ __forceinline__ void bcast_index(const Bcast& bc, int64_t i, int64_t& ia, int64_t& ib) {
    ia = 0;
    ib = 0;
    if (bc.narrow) {
        uint32_t j = (uint32_t)i, a = 0, b = 0;
#pragma unroll
        for (int d = MTL_MAX_RANK - 1; d >= 0; --d) {
            if (d < bc.rank) {
                const uint32_t s = (uint32_t)bc.shape[d];
                const uint32_t q = j / s;
                const uint32_t r = j - q * s;
                a += r * (uint32_t)bc.sa[d];
                b += r * (uint32_t)bc.sb[d];
                j = q;
            }
        }
        ia = a;
        ib = b;
        return;
    }
#pragma unroll
    for (int d = MTL_MAX_RANK - 1; d >= 0; --d) {
        if (d < bc.rank) {
            int64_t q = i / bc.shape[d];
            int64_t r = i - q * bc.shape[d];
            ia += r * bc.sa[d];
            ib += r * bc.sb[d];
            i = q;
        }
    }
}

__global__ void __launch_bounds__(kBlock) k_binary_bcast(float* __restrict__ out, const float* __restrict__ a,
                                                         const float* __restrict__ b, int64_t n, int op,
                                                         Bcast bc) {
    mtl_pdl_sync();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) {
        int64_t ia, ib;
        bcast_index(bc, i, ia, ib);
        out[i] = bin_apply(op, a[ia], b[ib]);
    }
}

// out[i] = a[i] op s  or  s op a[i], s read from device memory (the [1]-shaped operand)
__global__ void __launch_bounds__(kBlock) k_binary_scalar(float* __restrict__ out, const float* __restrict__ t,
                                                          const float* __restrict__ s, int64_t n, int op,
                                                          int scalar_first, int vec) {
    mtl_pdl_sync();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    float sv = __ldg(s);
    if (vec) {
        int64_t n4 = n >> 2;
        const float4* t4 = reinterpret_cast<const float4*>(t);
        float4* o4 = reinterpret_cast<float4*>(out);
        for (int64_t i = tid; i < n4; i += stride) {
            float4 v = t4[i];
            if (scalar_first) {
                v.x = bin_apply(op, sv, v.x); v.y = bin_apply(op, sv, v.y);
                v.z = bin_apply(op, sv, v.z); v.w = bin_apply(op, sv, v.w);
            } else {
                v.x = bin_apply(op, v.x, sv); v.y = bin_apply(op, v.y, sv);
                v.z = bin_apply(op, v.z, sv); v.w = bin_apply(op, v.w, sv);
            }
            o4[i] = v;
        }
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride)
            out[i] = scalar_first ? bin_apply(op, sv, t[i]) : bin_apply(op, t[i], sv);
    } else {
        for (int64_t i = tid; i < n; i += stride)
            out[i] = scalar_first ? bin_apply(op, sv, t[i]) : bin_apply(op, t[i], sv);
    }
}

// Local gradient of a binary op at broadcast index i (basics.mojo:46-219).
__device__ __forceinline__ float bin_bwd_value(int op, int tensor_id, float ug, float a, float b,
                                               int b_is_scalar) {
    switch (op) {
        case MTL_OP_ADD: return ug;
        case MTL_OP_SUB: return tensor_id == 0 ? ug : ug * -1.0f;
        case MTL_OP_MUL: return tensor_id == 0 ? ug * b : ug * a;
        default:
            if (tensor_id == 0) return ug / b;
            if (b_is_scalar) return (-1.0f / (b * b)) * a * ug;
            return -a / (b * b) * ug;
    }
}

// grad has the broadcast shape itself: one thread per element.
__global__ void __launch_bounds__(kBlock) k_binary_bwd_full(float* __restrict__ grad, const float* __restrict__ ug,
                                                            const float* __restrict__ a,
                                                            const float* __restrict__ b, int64_t n, int op,
                                                            int tensor_id, int b_is_scalar, int acc, Bcast bc) {
    mtl_pdl_sync();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) {
        int64_t ia, ib;
        bcast_index(bc, i, ia, ib);
        float av = a ? a[ia] : 0.0f, bv = b ? b[ib] : 0.0f;
        float r = bin_bwd_value(op, tensor_id, ug[i], av, bv, b_is_scalar);
        grad[i] = acc ? grad[i] + r : r;
    }
}

// Un-broadcast: grad element j sums the contributions of every broadcast index that maps to it.
// `keep` enumerates the operand's own axes (mixed radix -> j), `red` the axes it was broadcast over.
struct Unbcast {
    int n_keep, n_red;
    int narrow;  // the broadcast extent fits 32 bits
    int64_t keep_size[MTL_MAX_RANK], keep_ostride[MTL_MAX_RANK];  // size, stride in broadcast space
    int64_t red_size[MTL_MAX_RANK], red_ostride[MTL_MAX_RANK];
};

__device__ __forceinline__ int64_t unb_base(const Unbcast& u, int64_t j) {
    if (u.narrow) {
        uint32_t jj = (uint32_t)j, o = 0;
        for (int d = u.n_keep - 1; d >= 0; --d) {
            const uint32_t s = (uint32_t)u.keep_size[d];
            const uint32_t q = jj / s;
            o += (jj - q * s) * (uint32_t)u.keep_ostride[d];
            jj = q;
        }
        return o;
    }
    int64_t o = 0;
    for (int d = u.n_keep - 1; d >= 0; --d) {
        int64_t q = j / u.keep_size[d];
        o += (j - q * u.keep_size[d]) * u.keep_ostride[d];
        j = q;
    }
    return o;
}
__device__ __forceinline__ int64_t unb_red(const Unbcast& u, int64_t r) {
    if (u.narrow) {
        uint32_t rr = (uint32_t)r, o = 0;
        for (int d = u.n_red - 1; d >= 0; --d) {
            const uint32_t s = (uint32_t)u.red_size[d];
            const uint32_t q = rr / s;
            o += (rr - q * s) * (uint32_t)u.red_ostride[d];
            rr = q;
        }
        return o;
    }
    int64_t o = 0;
    for (int d = u.n_red - 1; d >= 0; --d) {
        int64_t q = r / u.red_size[d];
        o += (r - q * u.red_size[d]) * u.red_ostride[d];
        r = q;
    }
    return o;
}

// One block per grad element (long reductions, e.g. a bias gradient over the batch).
__global__ void __launch_bounds__(kBlock) k_binary_bwd_unb_block(float* __restrict__ grad,
                                                                 const float* __restrict__ ug,
                                                                 const float* __restrict__ a,
                                                                 const float* __restrict__ b, int64_t n_grad,
                                                                 int64_t n_red, int op, int tensor_id,
                                                                 int b_is_scalar, int acc, Bcast bc, Unbcast ub) {
    mtl_pdl_sync();
    __shared__ float warp_sums[kBlock / 32];
    for (int64_t j = blockIdx.x; j < n_grad; j += gridDim.x) {
        int64_t base = unb_base(ub, j);
        float s = 0.0f;
        for (int64_t r = threadIdx.x; r < n_red; r += blockDim.x) {
            int64_t i = base + unb_red(ub, r);
            int64_t ia, ib;
            bcast_index(bc, i, ia, ib);
            float av = a ? a[ia] : 0.0f, bv = b ? b[ib] : 0.0f;
            s += bin_bwd_value(op, tensor_id, ug[i], av, bv, b_is_scalar);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = s;
        __syncthreads();
        if (threadIdx.x < 32) {
            float t = threadIdx.x < kBlock / 32 ? warp_sums[threadIdx.x] : 0.0f;
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (threadIdx.x == 0) grad[j] = acc ? grad[j] + t : t;
        }
        __syncthreads();
    }
}

// The bias-gradient case of the kernel above without its general index arithmetic: ug is [R, C]
// (row-major), grad is [C], ADD or SUB.  Same assignment of rows to threads and same reduction tree,
// hence the same bits.
__global__ void __launch_bounds__(kBlock) k_unb_rows(float* __restrict__ grad, const float* __restrict__ ug, int64_t R,
                                                     int64_t C, float sign, int acc) {
    mtl_pdl_sync();
    __shared__ float warp_sums[kBlock / 32];
    for (int64_t j = blockIdx.x; j < C; j += gridDim.x) {
        float s = 0.0f;
        for (int64_t r = threadIdx.x; r < R; r += blockDim.x) s += sign * ug[r * C + j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = s;
        __syncthreads();
        if (threadIdx.x < 32) {
            float t = threadIdx.x < kBlock / 32 ? warp_sums[threadIdx.x] : 0.0f;
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (threadIdx.x == 0) grad[j] = acc ? grad[j] + t : t;
        }
        __syncthreads();
    }
}

// One thread per grad element (short reductions).
__global__ void __launch_bounds__(kBlock) k_binary_bwd_unb_thread(float* __restrict__ grad,
                                                                  const float* __restrict__ ug,
                                                                  const float* __restrict__ a,
                                                                  const float* __restrict__ b, int64_t n_grad,
                                                                  int64_t n_red, int op, int tensor_id,
                                                                  int b_is_scalar, int acc, Bcast bc, Unbcast ub) {
    mtl_pdl_sync();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t j = tid; j < n_grad; j += stride) {
        int64_t base = unb_base(ub, j);
        float s = 0.0f;
        for (int64_t r = 0; r < n_red; ++r) {
            int64_t i = base + unb_red(ub, r);
            int64_t ia, ib;
            bcast_index(bc, i, ia, ib);
            float av = a ? a[ia] : 0.0f, bv = b ? b[ib] : 0.0f;
            s += bin_bwd_value(op, tensor_id, ug[i], av, bv, b_is_scalar);
        }
        grad[j] = acc ? grad[j] + s : s;
    }
}

__global__ void __launch_bounds__(kBlock) k_fma(float* __restrict__ out, const float* __restrict__ a,
                                                const float* __restrict__ b, const float* __restrict__ c,
                                                int64_t n) {
    mtl_pdl_sync();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) out[i] = fmaf(a[i], b[i], c[i]);
}

inline int aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

// broadcast_shapes (tensorutils.mojo:89-127) + strides; returns false when not broadcastable.
bool make_bcast(int a_rank, const int64_t* a_shape, int b_rank, const int64_t* b_shape, Bcast* bc) {
    int rank = a_rank > b_rank ? a_rank : b_rank;
    if (rank > MTL_MAX_RANK || a_rank < 1 || b_rank < 1) return false;
    bc->rank = rank;
    int da = rank - a_rank, db = rank - b_rank;
    for (int d = 0; d < rank; ++d) {
        int64_t x = d >= da ? a_shape[d - da] : 1;
        int64_t y = d >= db ? b_shape[d - db] : 1;
        if (x != y && x != 1 && y != 1) return false;
        bc->shape[d] = x == 1 ? y : x;
    }
    int64_t st = 1;
    for (int d = rank - 1; d >= 0; --d) {
        int64_t x = d >= da ? a_shape[d - da] : 1;
        bc->sa[d] = (x != 1) ? st : 0;
        if (x != 1) st *= x;
    }
    st = 1;
    for (int d = rank - 1; d >= 0; --d) {
        int64_t y = d >= db ? b_shape[d - db] : 1;
        bc->sb[d] = (y != 1) ? st : 0;
        if (y != 1) st *= y;
    }
    for (int d = rank; d < MTL_MAX_RANK; ++d) { bc->shape[d] = 1; bc->sa[d] = 0; bc->sb[d] = 0; }
    bc->narrow = mtl_numel(rank, bc->shape) < (1ll << 31) ? 1 : 0;
    return true;
}

bool is_scalar_shape(int rank, const int64_t* shape) { return rank == 1 && shape[0] == 1; }
bool same_shape(int ra, const int64_t* a, int rb, const int64_t* b) {
    if (ra != rb) return false;
    for (int i = 0; i < ra; ++i)
        if (a[i] != b[i]) return false;
    return true;
}

bool unary_op_known(int op) {
    switch (op) {
        case MTL_OP_EXP: case MTL_OP_LOG: case MTL_OP_POW: case MTL_OP_SIGMOID: case MTL_OP_RELU:
        case MTL_OP_TANH: case MTL_OP_CLIP: case MTL_OP_LEAKYRELU: return true;
        default: return false;
    }
}

}  // namespace

namespace {
// out[b][c] = 1 when c == Int(labels[b]), else 0 (examples/mnist.mojo:92-97: labels arrive as fp32).
// A label outside [0, C) leaves its row all zeros; the reference would write outside the row.
__global__ void __launch_bounds__(kBlock) k_one_hot(float* __restrict__ out, const float* __restrict__ labels, int64_t B,
                                                    int64_t C) {
    mtl_pdl_sync();
    const int64_t n = B * C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t b = i / C, c = i - b * C;
        out[i] = (int64_t)labels[b] == c ? 1.0f : 0.0f;
    }
}
}  // namespace

extern "C" {

int32_t mtl_one_hot_f32(mtl_ctx* ctx, float* out, const float* labels, int64_t B, int64_t C) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, B >= 0 && C >= 1 && ((out && labels) || B == 0), "bad arguments to mtl_one_hot_f32");
    if (B == 0) return MTL_OK;
    int grid = mtl_grid_for(B * C, kBlock, ctx->sm_count, kCtasPerSm);
    mtl_launch_pdl(ctx, k_one_hot, dim3(grid), dim3(kBlock), (size_t)(0), out, labels, B, C);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_fill_f32(mtl_ctx* ctx, float* dptr, int64_t n, float value) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, n >= 0 && (dptr || n == 0), "bad arguments to mtl_fill_f32");
    if (n == 0) return MTL_OK;
    int grid = mtl_grid_for((n + 3) / 4, kBlock, ctx->sm_count, kCtasPerSm);
    mtl_launch_pdl(ctx, k_fill, dim3(grid), dim3(kBlock), (size_t)(0), dptr, n, value, aligned16(dptr));
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_copy_f32(mtl_ctx* ctx, float* dst, const float* src, int64_t n, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, n >= 0 && ((dst && src) || n == 0), "bad arguments to mtl_copy_f32");
    if (n == 0) return MTL_OK;
    if (!accumulate) {
        MTL_CUDA(ctx, cudaMemcpyAsync(dst, src, (size_t)n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        return MTL_OK;
    }
    int vec = aligned16(dst) && aligned16(src);
    int grid = mtl_grid_for((n + 3) / 4, kBlock, ctx->sm_count, kCtasPerSm);
    mtl_launch_pdl(ctx, k_map2<AddTo>, dim3(grid), dim3(kBlock), (size_t)(0), dst, dst, src, n, AddTo{}, vec, 0);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_unary_fwd(mtl_ctx* ctx, int32_t op, float* out, const float* in, int64_t n, float p0,
                      float p1) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, unary_op_known(op), "mtl_unary_fwd: op id %d is not a unary elementwise op", op);
    MTL_REQUIRE(ctx, n >= 0 && ((out && in) || n == 0), "bad arguments to mtl_unary_fwd");
    if (n == 0) return MTL_OK;
    int vec = aligned16(out) && aligned16(in);
    int grid = mtl_grid_for((n + 3) / 4, kBlock, ctx->sm_count, kCtasPerSm);
    mtl_launch_pdl(ctx, k_map1<UnaryFwd>, dim3(grid), dim3(kBlock), (size_t)(0), out, in, n, UnaryFwd{op, p0, p1}, vec);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_unary_bwd(mtl_ctx* ctx, int32_t op, float* grad, const float* ug, const float* in,
                      int64_t n, float p0, float p1, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, unary_op_known(op), "mtl_unary_bwd: op id %d is not a unary elementwise op", op);
    MTL_REQUIRE(ctx, n >= 0 && ((grad && ug && in) || n == 0), "bad arguments to mtl_unary_bwd");
    if (n == 0) return MTL_OK;
    int vec = aligned16(grad) && aligned16(ug) && aligned16(in);
    int grid = mtl_grid_for((n + 3) / 4, kBlock, ctx->sm_count, kCtasPerSm);
    mtl_launch_pdl(ctx, k_map2<UnaryBwd>, dim3(grid), dim3(kBlock), (size_t)(0), grad, in, ug, n, UnaryBwd{op, p0, p1}, vec, accumulate ? 1 : 0);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_binary_fwd(mtl_ctx* ctx, int32_t op, float* out, const float* a, const float* b,
                       int32_t a_rank, const int64_t* a_shape, int32_t b_rank, const int64_t* b_shape) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, op >= MTL_OP_ADD && op <= MTL_OP_DIV, "mtl_binary_fwd: op id %d is not ADD/SUB/MUL/DIV", op);
    MTL_REQUIRE(ctx, out && a && b && a_shape && b_shape, "null pointer in mtl_binary_fwd");
    Bcast bc;
    MTL_REQUIRE(ctx, make_bcast(a_rank, a_shape, b_rank, b_shape, &bc),
                "shapes cannot be broadcast together");
    int64_t n = mtl_numel(bc.rank, bc.shape);
    if (n == 0) return MTL_OK;
    // dispatch order of elwise_op (tensorutils.mojo:263-274)
    if (is_scalar_shape(b_rank, b_shape) || is_scalar_shape(a_rank, a_shape)) {
        int scalar_first = !is_scalar_shape(b_rank, b_shape);
        const float* t = scalar_first ? b : a;
        const float* s = scalar_first ? a : b;
        int vec = aligned16(out) && aligned16(t);
        int grid = mtl_grid_for((n + 3) / 4, kBlock, ctx->sm_count, kCtasPerSm);
        mtl_launch_pdl(ctx, k_binary_scalar, dim3(grid), dim3(kBlock), (size_t)(0), out, t, s, n, op, scalar_first, vec);
    } else if (same_shape(a_rank, a_shape, b_rank, b_shape)) {
        int vec = aligned16(out) && aligned16(a) && aligned16(b);
        int grid = mtl_grid_for((n + 3) / 4, kBlock, ctx->sm_count, kCtasPerSm);
        mtl_launch_pdl(ctx, k_map2<BinF>, dim3(grid), dim3(kBlock), (size_t)(0), out, a, b, n, BinF{op}, vec, 0);
    } else {
        int grid = mtl_grid_for(n, kBlock, ctx->sm_count, kCtasPerSm);
        mtl_launch_pdl(ctx, k_binary_bcast, dim3(grid), dim3(kBlock), (size_t)(0), out, a, b, n, op, bc);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_binary_bwd(mtl_ctx* ctx, int32_t op, int32_t tensor_id, float* grad, const float* ug,
                       const float* a, const float* b, int32_t a_rank, const int64_t* a_shape,
                       int32_t b_rank, const int64_t* b_shape, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, op >= MTL_OP_ADD && op <= MTL_OP_DIV, "mtl_binary_bwd: op id %d is not ADD/SUB/MUL/DIV", op);
    MTL_REQUIRE(ctx, tensor_id == 0 || tensor_id == 1, "tensor_id must be 0 or 1");
    MTL_REQUIRE(ctx, grad && ug && a_shape && b_shape, "null pointer in mtl_binary_bwd");
    bool need_a = (op == MTL_OP_MUL && tensor_id == 1) || (op == MTL_OP_DIV && tensor_id == 1);
    bool need_b = (op == MTL_OP_MUL && tensor_id == 0) || op == MTL_OP_DIV;
    MTL_REQUIRE(ctx, (!need_a || a) && (!need_b || b), "operand needed by this gradient is null");
    Bcast bc;
    MTL_REQUIRE(ctx, make_bcast(a_rank, a_shape, b_rank, b_shape, &bc), "shapes cannot be broadcast together");
    int64_t n = mtl_numel(bc.rank, bc.shape);
    if (n == 0) return MTL_OK;
    int g_rank = tensor_id == 0 ? a_rank : b_rank;
    const int64_t* g_shape = tensor_id == 0 ? a_shape : b_shape;
    int64_t n_grad = mtl_numel(g_rank, g_shape);
    int b_is_scalar = is_scalar_shape(b_rank, b_shape);
    int acc = accumulate ? 1 : 0;

    if (n_grad == n) {
        // grad already has the broadcast extent: accumulate_op[add] (tensorutils.mojo:469-470)
        int grid = mtl_grid_for(n, kBlock, ctx->sm_count, kCtasPerSm);
        mtl_launch_pdl(ctx, k_binary_bwd_full, dim3(grid), dim3(kBlock), (size_t)(0), grad, ug, a, b, n, op, tensor_id, b_is_scalar, acc, bc);
        MTL_LAUNCHED(ctx);
        return MTL_OK;
    }
    // un-broadcast (tensorutils.mojo:473-487)
    Unbcast ub;
    ub.n_keep = 0;
    ub.n_red = 0;
    ub.narrow = bc.narrow;
    int64_t ostride[MTL_MAX_RANK];
    int64_t st = 1;
    for (int d = bc.rank - 1; d >= 0; --d) { ostride[d] = st; st *= bc.shape[d]; }
    const int64_t* gs = tensor_id == 0 ? bc.sa : bc.sb;
    int64_t n_red = 1;
    for (int d = 0; d < bc.rank; ++d) {
        if (bc.shape[d] == 1) continue;
        if (gs[d] != 0) {
            ub.keep_size[ub.n_keep] = bc.shape[d];
            ub.keep_ostride[ub.n_keep++] = ostride[d];
        } else {
            ub.red_size[ub.n_red] = bc.shape[d];
            ub.red_ostride[ub.n_red++] = ostride[d];
            n_red *= bc.shape[d];
        }
    }
    if (n_red >= 128 && (op == MTL_OP_ADD || op == MTL_OP_SUB) && ub.n_keep == 1 && ub.n_red == 1 &&
        ub.keep_ostride[0] == 1 && ub.red_ostride[0] == ub.keep_size[0]) {
        // a bias gradient: column sums of a row-major [rows, n_grad] upper gradient
        const float sign = (op == MTL_OP_SUB && tensor_id == 1) ? -1.0f : 1.0f;
        int grid = (int)(n_grad < (int64_t)ctx->sm_count * kCtasPerSm ? n_grad : (int64_t)ctx->sm_count * kCtasPerSm);
        mtl_launch_pdl(ctx, k_unb_rows, dim3(grid), dim3(kBlock), (size_t)(0), grad, ug, n_red, n_grad, sign, acc);
        MTL_LAUNCHED(ctx);
        return MTL_OK;
    }
    if (n_red >= 128) {
        int grid = (int)(n_grad < (int64_t)ctx->sm_count * kCtasPerSm ? n_grad : (int64_t)ctx->sm_count * kCtasPerSm);
        mtl_launch_pdl(ctx, k_binary_bwd_unb_block, dim3(grid), dim3(kBlock), (size_t)(0), grad, ug, a, b, n_grad, n_red, op, tensor_id,
                                                                  b_is_scalar, acc, bc, ub);
    } else {
        int grid = mtl_grid_for(n_grad, kBlock, ctx->sm_count, kCtasPerSm);
        mtl_launch_pdl(ctx, k_binary_bwd_unb_thread, dim3(grid), dim3(kBlock), (size_t)(0), grad, ug, a, b, n_grad, n_red, op, tensor_id,
                                                                   b_is_scalar, acc, bc, ub);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_fma_fwd(mtl_ctx* ctx, float* out, const float* a, const float* b, const float* c, int64_t n) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, n >= 0 && ((out && a && b && c) || n == 0), "bad arguments to mtl_fma_fwd");
    if (n == 0) return MTL_OK;
    int grid = mtl_grid_for(n, kBlock, ctx->sm_count, kCtasPerSm);
    mtl_launch_pdl(ctx, k_fma, dim3(grid), dim3(kBlock), (size_t)(0), out, a, b, c, n);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_fma_bwd(mtl_ctx* ctx, int32_t tensor_id, float* grad, const float* ug, const float* a,
                    const float* b, int64_t n, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, tensor_id >= 0 && tensor_id <= 2, "tensor_id must be 0, 1 or 2");
    MTL_REQUIRE(ctx, n >= 0 && ((grad && ug) || n == 0), "bad arguments to mtl_fma_bwd");
    if (n == 0) return MTL_OK;
    if (tensor_id == 2) return mtl_copy_f32(ctx, grad, ug, n, accumulate);
    const float* other = tensor_id == 0 ? b : a;
    MTL_REQUIRE(ctx, other, "operand needed by this gradient is null");
    int vec = aligned16(grad) && aligned16(ug) && aligned16(other);
    int grid = mtl_grid_for((n + 3) / 4, kBlock, ctx->sm_count, kCtasPerSm);
    mtl_launch_pdl(ctx, k_map2<BinF>, dim3(grid), dim3(kBlock), (size_t)(0), grad, ug, other, n, BinF{MTL_OP_MUL}, vec, accumulate ? 1 : 0);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

}  // extern "C"
