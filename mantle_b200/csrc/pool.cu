// MAXPOOL2D forward (value + argmax index) and backward.  HBM-bound: the common 2x2 stride-2 case
// reads float4 pairs and writes float2 values / int2 indices; every other geometry takes the
// generic window scan.  Scan order, -inf start and the strict `>` update follow
// mantle/autograd/ops/pool.mojo:62-100 so that the selected index is the reference's.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kBlock = 256;

struct PoolGeom {
    int N, C, H, W, OH, OW;
    int R, S, ph, pw, sh, sw, dh, dw;
};

__device__ __forceinline__ void window_argmax(const float* __restrict__ plane, const PoolGeom& g, int oh, int ow,
                                              float& best, int& best_idx) {
    best = -INFINITY;
    best_idx = -1;
    int ih0 = oh * g.sh - g.ph, iw0 = ow * g.sw - g.pw;
    for (int r = 0; r < g.R; ++r) {
        int ih = ih0 + r * g.dh;
        if (ih < 0 || ih >= g.H) continue;
        for (int s = 0; s < g.S; ++s) {
            int iw = iw0 + s * g.dw;
            if (iw < 0 || iw >= g.W) continue;
            float v = plane[ih * g.W + iw];
            if (v > best) {
                best = v;
                best_idx = ih * g.W + iw;
            }
        }
    }
}

__global__ void __launch_bounds__(kBlock) k_pool_fwd_generic(float* __restrict__ Y, int32_t* __restrict__ idx,
                                                             const float* __restrict__ X, PoolGeom g, int64_t n_out) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int plane_out = g.OH * g.OW;
    for (int64_t o = tid; o < n_out; o += stride) {
        int64_t pl = o / plane_out;
        int rem = (int)(o - pl * plane_out);
        int oh = rem / g.OW, ow = rem - oh * g.OW;
        float best;
        int bi;
        window_argmax(X + pl * (int64_t)g.H * g.W, g, oh, ow, best, bi);
        Y[o] = best;
        if (idx) idx[o] = bi;
    }
}

// 2x2 window, stride 2, no padding, no dilation, even W: each thread produces two adjacent outputs
// from two float4 row segments.
__global__ void __launch_bounds__(kBlock) k_pool_fwd_2x2(float* __restrict__ Y, int32_t* __restrict__ idx,
                                                         const float* __restrict__ X, int H, int W, int OH, int OW,
                                                         int64_t n_pairs) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int pairs_per_row = OW >> 1;
    for (int64_t p = tid; p < n_pairs; p += stride) {
        int64_t row = p / pairs_per_row;  // (plane, oh)
        int pc = (int)(p - row * pairs_per_row);
        int64_t pl = row / OH;
        int oh = (int)(row - pl * OH);
        const float* base = X + pl * (int64_t)H * W + (int64_t)(2 * oh) * W + 4 * pc;
        float4 a = *reinterpret_cast<const float4*>(base);
        float4 b = *reinterpret_cast<const float4*>(base + W);
        int i00 = (2 * oh) * W + 4 * pc;
        float m0 = -INFINITY, m1 = -INFINITY;
        int j0 = -1, j1 = -1;
        if (a.x > m0) { m0 = a.x; j0 = i00; }
        if (a.y > m0) { m0 = a.y; j0 = i00 + 1; }
        if (b.x > m0) { m0 = b.x; j0 = i00 + W; }
        if (b.y > m0) { m0 = b.y; j0 = i00 + W + 1; }
        if (a.z > m1) { m1 = a.z; j1 = i00 + 2; }
        if (a.w > m1) { m1 = a.w; j1 = i00 + 3; }
        if (b.z > m1) { m1 = b.z; j1 = i00 + W + 2; }
        if (b.w > m1) { m1 = b.w; j1 = i00 + W + 3; }
        int64_t o = row * OW + 2 * pc;
        *reinterpret_cast<float2*>(Y + o) = make_float2(m0, m1);
        if (idx) *reinterpret_cast<int2*>(idx + o) = make_int2(j0, j1);
    }
}

// Backward for windows that never overlap (stride >= dilated extent): every input element belongs to
// at most one window, so plain read-modify-write is race free.  `dX` must already hold zeros (or the
// running gradient when accumulating).
template <bool FROM_IDX, bool ATOMIC>
__global__ void __launch_bounds__(kBlock) k_pool_bwd(float* __restrict__ dX, const float* __restrict__ ug,
                                                     const float* __restrict__ X, const int32_t* __restrict__ idx,
                                                     const float* __restrict__ relu_of, PoolGeom g, int64_t n_out) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int plane_out = g.OH * g.OW;
    for (int64_t o = tid; o < n_out; o += stride) {
        int64_t pl = o / plane_out;
        int bi;
        if (FROM_IDX) {
            bi = idx[o];
        } else {
            int rem = (int)(o - pl * plane_out);
            int oh = rem / g.OW, ow = rem - oh * g.OW;
            float best;
            window_argmax(X + pl * (int64_t)g.H * g.W, g, oh, ow, best, bi);
        }
        if (bi < 0 || bi >= g.H * g.W) continue;  // no element exceeded -inf: nothing to route
        float* dst = dX + pl * (int64_t)g.H * g.W + bi;
        // fused RELU.backward of the layer below: the selected element is the pooled value itself
        const float u = relu_of ? (relu_of[o] > 0.0f ? 1.0f : 0.0f) * ug[o] : ug[o];
        if (ATOMIC) atomicAdd(dst, u);
        else *dst += u;
    }
}

// 2x2 stride-2 backward that writes every input element exactly once (no zero-fill pass needed
// when not accumulating): each thread owns two windows = a 2x4 input patch.
template <bool FROM_IDX>
__global__ void __launch_bounds__(kBlock) k_pool_bwd_2x2(float* __restrict__ dX, const float* __restrict__ ug,
                                                         const float* __restrict__ X, const int32_t* __restrict__ idx,
                                                         const float* __restrict__ relu_of, int H, int W, int OH,
                                                         int OW, int64_t n_pairs, int acc) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int pairs_per_row = OW >> 1;
    for (int64_t p = tid; p < n_pairs; p += stride) {
        int64_t row = p / pairs_per_row;
        int pc = (int)(p - row * pairs_per_row);
        int64_t pl = row / OH;
        int oh = (int)(row - pl * OH);
        int i00 = (2 * oh) * W + 4 * pc;
        int64_t o = row * OW + 2 * pc;
        int j0, j1;
        if (FROM_IDX) {
            int2 j = *reinterpret_cast<const int2*>(idx + o);
            j0 = j.x;
            j1 = j.y;
        } else {
            const float* base = X + pl * (int64_t)H * W + i00;
            float4 a = *reinterpret_cast<const float4*>(base);
            float4 b = *reinterpret_cast<const float4*>(base + W);
            float m0 = -INFINITY, m1 = -INFINITY;
            j0 = -1; j1 = -1;
            if (a.x > m0) { m0 = a.x; j0 = i00; }
            if (a.y > m0) { m0 = a.y; j0 = i00 + 1; }
            if (b.x > m0) { m0 = b.x; j0 = i00 + W; }
            if (b.y > m0) { m0 = b.y; j0 = i00 + W + 1; }
            if (a.z > m1) { m1 = a.z; j1 = i00 + 2; }
            if (a.w > m1) { m1 = a.w; j1 = i00 + 3; }
            if (b.z > m1) { m1 = b.z; j1 = i00 + W + 2; }
            if (b.w > m1) { m1 = b.w; j1 = i00 + W + 3; }
        }
        float2 u = *reinterpret_cast<const float2*>(ug + o);
        if (relu_of) {
            const float2 y = *reinterpret_cast<const float2*>(relu_of + o);
            u.x = (y.x > 0.0f ? 1.0f : 0.0f) * u.x;
            u.y = (y.y > 0.0f ? 1.0f : 0.0f) * u.y;
        }
        float4 ra, rb;
        ra.x = j0 == i00 ? u.x : 0.0f;
        ra.y = j0 == i00 + 1 ? u.x : 0.0f;
        rb.x = j0 == i00 + W ? u.x : 0.0f;
        rb.y = j0 == i00 + W + 1 ? u.x : 0.0f;
        ra.z = j1 == i00 + 2 ? u.y : 0.0f;
        ra.w = j1 == i00 + 3 ? u.y : 0.0f;
        rb.z = j1 == i00 + W + 2 ? u.y : 0.0f;
        rb.w = j1 == i00 + W + 3 ? u.y : 0.0f;
        float* d0 = dX + pl * (int64_t)H * W + i00;
        if (acc) {
            float4 oa = *reinterpret_cast<const float4*>(d0);
            float4 ob = *reinterpret_cast<const float4*>(d0 + W);
            ra.x += oa.x; ra.y += oa.y; ra.z += oa.z; ra.w += oa.w;
            rb.x += ob.x; rb.y += ob.y; rb.z += ob.z; rb.w += ob.w;
        }
        *reinterpret_cast<float4*>(d0) = ra;
        *reinterpret_cast<float4*>(d0 + W) = rb;
    }
}

// The same 2x2 / stride 2 case for any even W (e.g. 14): one window per thread, float2 rows.
__global__ void __launch_bounds__(kBlock) k_pool_fwd_2x2_one(float* __restrict__ Y, int32_t* __restrict__ idx,
                                                             const float* __restrict__ X, int H, int W, int OH, int OW,
                                                             int64_t n_out) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t o = tid; o < n_out; o += stride) {
        int64_t row = o / OW;  // (plane, oh)
        int ow = (int)(o - row * OW);
        int64_t pl = row / OH;
        int oh = (int)(row - pl * OH);
        int i00 = (2 * oh) * W + 2 * ow;
        const float* base = X + pl * (int64_t)H * W + i00;
        float2 a = *reinterpret_cast<const float2*>(base);
        float2 b = *reinterpret_cast<const float2*>(base + W);
        float m = -INFINITY;
        int j = -1;
        if (a.x > m) { m = a.x; j = i00; }
        if (a.y > m) { m = a.y; j = i00 + 1; }
        if (b.x > m) { m = b.x; j = i00 + W; }
        if (b.y > m) { m = b.y; j = i00 + W + 1; }
        Y[o] = m;
        if (idx) idx[o] = j;
    }
}

template <bool FROM_IDX>
__global__ void __launch_bounds__(kBlock) k_pool_bwd_2x2_one(float* __restrict__ dX, const float* __restrict__ ug,
                                                             const float* __restrict__ X, const int32_t* __restrict__ idx,
                                                             const float* __restrict__ relu_of, int H, int W, int OH,
                                                             int OW, int64_t n_out, int acc) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t o = tid; o < n_out; o += stride) {
        int64_t row = o / OW;
        int ow = (int)(o - row * OW);
        int64_t pl = row / OH;
        int oh = (int)(row - pl * OH);
        int i00 = (2 * oh) * W + 2 * ow;
        int j;
        if (FROM_IDX) {
            j = idx[o];
        } else {
            const float* base = X + pl * (int64_t)H * W + i00;
            float2 a = *reinterpret_cast<const float2*>(base);
            float2 b = *reinterpret_cast<const float2*>(base + W);
            float m = -INFINITY;
            j = -1;
            if (a.x > m) { m = a.x; j = i00; }
            if (a.y > m) { m = a.y; j = i00 + 1; }
            if (b.x > m) { m = b.x; j = i00 + W; }
            if (b.y > m) { m = b.y; j = i00 + W + 1; }
        }
        float u = ug[o];
        if (relu_of) u = (relu_of[o] > 0.0f ? 1.0f : 0.0f) * u;
        float2 ra, rb;
        ra.x = j == i00 ? u : 0.0f;
        ra.y = j == i00 + 1 ? u : 0.0f;
        rb.x = j == i00 + W ? u : 0.0f;
        rb.y = j == i00 + W + 1 ? u : 0.0f;
        float* d0 = dX + pl * (int64_t)H * W + i00;
        if (acc) {
            float2 oa = *reinterpret_cast<const float2*>(d0);
            float2 ob = *reinterpret_cast<const float2*>(d0 + W);
            ra.x += oa.x; ra.y += oa.y; rb.x += ob.x; rb.y += ob.y;
        }
        *reinterpret_cast<float2*>(d0) = ra;
        *reinterpret_cast<float2*>(d0 + W) = rb;
    }
}

int32_t make_geom(mtl_ctx* ctx, const mtl_conv2d_desc* d, PoolGeom* g) {
    MTL_REQUIRE(ctx, d, "null descriptor");
    int32_t OH, OW;
    if (mtl_conv2d_out_shape(d, &OH, &OW) != MTL_OK)
        return mtl_set_error(ctx, MTL_ERR_INVALID, "pooling geometry gives an empty or invalid output");
    g->N = d->N; g->C = d->C; g->H = d->H; g->W = d->W; g->OH = OH; g->OW = OW;
    g->R = d->R; g->S = d->S; g->ph = d->pad[0]; g->pw = d->pad[1];
    g->sh = d->stride[0]; g->sw = d->stride[1]; g->dh = d->dilation[0]; g->dw = d->dilation[1];
    MTL_REQUIRE(ctx, (int64_t)d->H * d->W < (1ll << 31), "input plane too large for int32 indices");
    return MTL_OK;
}

bool is_fast_2x2(const PoolGeom& g, const void* X, const void* Y, const void* aux) {
    // full coverage of the input needs even H and W; float4 rows need W % 4 == 0 and aligned bases
    return g.R == 2 && g.S == 2 && g.sh == 2 && g.sw == 2 && g.ph == 0 && g.pw == 0 && g.dh == 1 && g.dw == 1 &&
           (g.W % 4) == 0 && (g.H % 2) == 0 && (((uintptr_t)X) & 15u) == 0 && (((uintptr_t)Y) & 7u) == 0 &&
           (((uintptr_t)aux) & 7u) == 0;
}

bool is_fast_2x2_one(const PoolGeom& g, const void* X) {
    // full coverage of the input needs even H and W; float2 rows need an 8-byte aligned base
    return g.R == 2 && g.S == 2 && g.sh == 2 && g.sw == 2 && g.ph == 0 && g.pw == 0 && g.dh == 1 && g.dw == 1 &&
           (g.W % 2) == 0 && (g.H % 2) == 0 && (((uintptr_t)X) & 7u) == 0;
}

int32_t pool_bwd(mtl_ctx* ctx, float* dX, const float* ug, const float* X, const int32_t* idx, const float* relu_of,
                 const mtl_conv2d_desc* d, int32_t accumulate) {
    PoolGeom g;
    int32_t rc = make_geom(ctx, d, &g);
    if (rc) return rc;
    MTL_REQUIRE(ctx, dX && ug && (X || idx), "null pointer in max-pool backward");
    int64_t planes = (int64_t)g.N * g.C;
    int64_t n_out = planes * g.OH * g.OW;
    int64_t n_in = planes * g.H * g.W;
    // the two-window kernel reads ug and the pooled values (relu_of) as float2: both need 8-byte alignment
    if (is_fast_2x2(g, idx ? (const void*)dX : (const void*)X, ug, idx) && (((uintptr_t)dX) & 15u) == 0 &&
        (((uintptr_t)relu_of) & 7u) == 0) {
        int64_t n_pairs = n_out / 2;
        int grid = mtl_grid_for(n_pairs, kBlock, ctx->sm_count, 8);
        if (idx)
            k_pool_bwd_2x2<true><<<grid, kBlock, 0, ctx->stream>>>(dX, ug, X, idx, relu_of, g.H, g.W, g.OH, g.OW, n_pairs, accumulate ? 1 : 0);
        else
            k_pool_bwd_2x2<false><<<grid, kBlock, 0, ctx->stream>>>(dX, ug, X, idx, relu_of, g.H, g.W, g.OH, g.OW, n_pairs, accumulate ? 1 : 0);
        MTL_LAUNCHED(ctx);
        return MTL_OK;
    }
    if (is_fast_2x2_one(g, idx ? (const void*)dX : (const void*)X) && (((uintptr_t)dX) & 7u) == 0) {
        int grid = mtl_grid_for(n_out, kBlock, ctx->sm_count, 8);
        if (idx)
            k_pool_bwd_2x2_one<true><<<grid, kBlock, 0, ctx->stream>>>(dX, ug, X, idx, relu_of, g.H, g.W, g.OH, g.OW, n_out, accumulate ? 1 : 0);
        else
            k_pool_bwd_2x2_one<false><<<grid, kBlock, 0, ctx->stream>>>(dX, ug, X, idx, relu_of, g.H, g.W, g.OH, g.OW, n_out, accumulate ? 1 : 0);
        MTL_LAUNCHED(ctx);
        return MTL_OK;
    }
    if (!accumulate) MTL_CUDA(ctx, cudaMemsetAsync(dX, 0, (size_t)n_in * 4, ctx->stream));
    bool overlap = g.sh < (g.R - 1) * g.dh + 1 || g.sw < (g.S - 1) * g.dw + 1;
    int grid = mtl_grid_for(n_out, kBlock, ctx->sm_count, 8);
    if (idx) {
        if (overlap) k_pool_bwd<true, true><<<grid, kBlock, 0, ctx->stream>>>(dX, ug, X, idx, relu_of, g, n_out);
        else k_pool_bwd<true, false><<<grid, kBlock, 0, ctx->stream>>>(dX, ug, X, idx, relu_of, g, n_out);
    } else {
        if (overlap) k_pool_bwd<false, true><<<grid, kBlock, 0, ctx->stream>>>(dX, ug, X, idx, relu_of, g, n_out);
        else k_pool_bwd<false, false><<<grid, kBlock, 0, ctx->stream>>>(dX, ug, X, idx, relu_of, g, n_out);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

}  // namespace

extern "C" {

int32_t mtl_conv2d_out_shape(const mtl_conv2d_desc* d, int32_t* OH, int32_t* OW) {
    if (!d || !OH || !OW) return MTL_ERR_INVALID;
    if (d->N < 1 || d->C < 1 || d->H < 1 || d->W < 1 || d->R < 1 || d->S < 1 || d->stride[0] < 1 ||
        d->stride[1] < 1 || d->dilation[0] < 1 || d->dilation[1] < 1 || d->pad[0] < 0 || d->pad[1] < 0)
        return MTL_ERR_INVALID;
    // get_result_shape, mantle/autograd/ops/conv.mojo:39-56 (floor division)
    int64_t nx = (int64_t)d->H + 2 * d->pad[0] - (int64_t)d->dilation[0] * (d->R - 1) - 1;
    int64_t ny = (int64_t)d->W + 2 * d->pad[1] - (int64_t)d->dilation[1] * (d->S - 1) - 1;
    if (nx < 0 || ny < 0) return MTL_ERR_INVALID;
    *OH = (int32_t)(nx / d->stride[0] + 1);
    *OW = (int32_t)(ny / d->stride[1] + 1);
    return MTL_OK;
}

int32_t mtl_maxpool2d_fwd(mtl_ctx* ctx, float* Y, int32_t* idx, const float* X, const mtl_conv2d_desc* d) {
    MTL_CHECK_CTX(ctx);
    PoolGeom g;
    int32_t rc = make_geom(ctx, d, &g);
    if (rc) return rc;
    MTL_REQUIRE(ctx, Y && X, "null pointer in mtl_maxpool2d_fwd");
    int64_t planes = (int64_t)g.N * g.C;
    int64_t n_out = planes * g.OH * g.OW;
    if (is_fast_2x2(g, X, Y, idx)) {
        int64_t n_pairs = n_out / 2;
        int grid = mtl_grid_for(n_pairs, kBlock, ctx->sm_count, 8);
        k_pool_fwd_2x2<<<grid, kBlock, 0, ctx->stream>>>(Y, idx, X, g.H, g.W, g.OH, g.OW, n_pairs);
    } else if (is_fast_2x2_one(g, X)) {
        int grid = mtl_grid_for(n_out, kBlock, ctx->sm_count, 8);
        k_pool_fwd_2x2_one<<<grid, kBlock, 0, ctx->stream>>>(Y, idx, X, g.H, g.W, g.OH, g.OW, n_out);
    } else {
        int grid = mtl_grid_for(n_out, kBlock, ctx->sm_count, 8);
        k_pool_fwd_generic<<<grid, kBlock, 0, ctx->stream>>>(Y, idx, X, g, n_out);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_maxpool2d_bwd(mtl_ctx* ctx, float* dX, const float* ug, const float* X, const mtl_conv2d_desc* d,
                          int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, X, "null input in mtl_maxpool2d_bwd");
    return pool_bwd(ctx, dX, ug, X, nullptr, nullptr, d, accumulate);
}

int32_t mtl_maxpool2d_bwd_idx(mtl_ctx* ctx, float* dX, const float* ug, const int32_t* idx,
                              const mtl_conv2d_desc* d, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, idx, "null indices in mtl_maxpool2d_bwd_idx");
    return pool_bwd(ctx, dX, ug, nullptr, idx, nullptr, d, accumulate);
}

int32_t mtl_maxpool2d_bwd_idx_act(mtl_ctx* ctx, float* dX, const float* ug, const int32_t* idx, const float* pooled,
                                  const mtl_conv2d_desc* d, int32_t act_op, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, idx, "null indices in mtl_maxpool2d_bwd_idx_act");
    MTL_REQUIRE(ctx, act_op == MTL_OP_RELU || act_op < 0, "mtl_maxpool2d_bwd_idx_act fuses RELU only (act_op %d)", act_op);
    MTL_REQUIRE(ctx, act_op < 0 || pooled, "the fused RELU gradient needs the pooled output");
    return pool_bwd(ctx, dX, ug, nullptr, idx, act_op == MTL_OP_RELU ? pooled : nullptr, d, accumulate);
}

}  // extern "C"
