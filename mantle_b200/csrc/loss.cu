// nn.CrossEntropyLoss as two launches.  The reference builds the loss from nine operator nodes
// (nn/loss.mojo:45-61 over nn/activations.mojo:94-108):
//     mx = MAX(x, 1); xm = x - mx; ex = EXP(xm); sm = SUM(ex, 1); lg = LOG(sm); ls = xm - lg;
//     t = y * ls; ret = SUM(t); loss = ret * (-1 / B)
// and its backward from the nine backward calls in reverse.  On [B, C] logits with a small C every
// one of those is a launch that moves a few kilobytes; here one thread owns a row and performs the
// same fp32 operations in the same order (only the order of the final sum over rows differs).
#include <float.h>

#include "common.cuh"

namespace {

constexpr int kLossBlock = 1024;

// Gradient of one row of logits for an upper gradient of 1 on the loss (overwrites or adds to gr):
//   d ls = y * scale                         (SUM.backward, MUL.backward)
//   d lg = -sum_c d ls                       (SUB.backward, operand 1, summed over the broadcast axis)
//   d sm = d lg / sm                         (LOG.backward)
//   d xm = d ls + d sm * ex                  (SUB.backward operand 0, then EXP.backward added to it)
//   d mx = -sum_c d xm                       (SUB.backward, operand 1)
//   d x  = d xm + [x == mx] * d mx / ties    (SUB.backward operand 0, then MAX.backward added to it)
__device__ __forceinline__ void cross_entropy_row_grad(float* __restrict__ gr, const float* __restrict__ xr,
                                                       const float* __restrict__ yr, int C, float scale, float mx,
                                                       int accumulate) {
    float sm = 0.0f, ties = 0.0f, dlg = 0.0f;
    for (int c = 0; c < C; ++c) {
        sm += expf(xr[c] - mx);
        ties += xr[c] == mx ? 1.0f : 0.0f;
        dlg += yr[c] * scale;
    }
    dlg = -dlg;
    const float dsm = dlg / sm;
    float dmx = 0.0f;
    for (int c = 0; c < C; ++c) dmx += yr[c] * scale + expf(xr[c] - mx) * dsm;
    dmx = -dmx;
    const float tie_share = (1.0f / ties) * dmx;
    for (int c = 0; c < C; ++c) {
        const float dxm = yr[c] * scale + expf(xr[c] - mx) * dsm;
        const float r = dxm + (xr[c] == mx ? tie_share : 0.0f);
        gr[c] = accumulate ? gr[c] + r : r;
    }
}

// Block 0: the loss.  Thread t owns rows t, t + 1024, ...; the per-thread sums are combined by a tree.  With
// `dx` the launch has more blocks, and block b > 0 writes the gradient of rows (b - 1) * 1024 + t (what
// k_cross_entropy_bwd computes), so that a training step spends one launch on the loss instead of two.
__global__ void __launch_bounds__(kLossBlock) k_cross_entropy_fwd(float* __restrict__ loss, float* __restrict__ dx,
                                                                  const float* __restrict__ x,
                                                                  const float* __restrict__ y, int B, int C, float scale) {
    mtl_pdl_sync();
    if (blockIdx.x > 0) {
        const int b = ((int)blockIdx.x - 1) * kLossBlock + (int)threadIdx.x;
        if (b < B) {
            const float* xr = x + (int64_t)b * C;
            float mx = -FLT_MAX;
            for (int c = 0; c < C; ++c) mx = fmaxf(mx, xr[c]);
            cross_entropy_row_grad(dx + (int64_t)b * C, xr, y + (int64_t)b * C, C, scale, mx, 0);
        }
        return;
    }
    __shared__ float part[kLossBlock];
    float acc = 0.0f;
    for (int b = threadIdx.x; b < B; b += kLossBlock) {
        const float* xr = x + (int64_t)b * C;
        const float* yr = y + (int64_t)b * C;
        float mx = -FLT_MAX;                              // MAX.forward along the axis
        for (int c = 0; c < C; ++c) mx = fmaxf(mx, xr[c]);
        float sm = 0.0f;                                  // SUM(EXP(x - mx)) in ascending order
        for (int c = 0; c < C; ++c) sm += expf(xr[c] - mx);
        const float lg = logf(sm);
        for (int c = 0; c < C; ++c) acc += yr[c] * ((xr[c] - mx) - lg);
    }
    part[threadIdx.x] = acc;
    __syncthreads();
    for (int s = kLossBlock / 2; s > 0; s >>= 1) {
        if ((int)threadIdx.x < s) part[threadIdx.x] += part[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) loss[0] = part[0] * scale;
}

// Gradient of the logits for an upper gradient of 1 on the loss; one thread per row.
__global__ void __launch_bounds__(256) k_cross_entropy_bwd(float* __restrict__ dx, const float* __restrict__ x,
                                                           const float* __restrict__ y, int B, int C, float scale,
                                                           int accumulate) {
    mtl_pdl_sync();
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    const float* xr = x + (int64_t)b * C;
    const float* yr = y + (int64_t)b * C;
    float* gr = dx + (int64_t)b * C;
    float mx = -FLT_MAX;
    for (int c = 0; c < C; ++c) mx = fmaxf(mx, xr[c]);
    cross_entropy_row_grad(gr, xr, yr, C, scale, mx, accumulate);
}

}  // namespace

extern "C" {

int32_t mtl_cross_entropy_fwd(mtl_ctx* ctx, float* loss, const float* logits, const float* y_true, int64_t B,
                              int64_t C, float scale) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, loss && logits && y_true, "null pointer in mtl_cross_entropy_fwd");
    MTL_REQUIRE(ctx, B >= 1 && C >= 1 && B * C <= MTL_CROSS_ENTROPY_MAX_ELEMENTS,
                "mtl_cross_entropy_fwd handles up to %lld logits, got %lld x %lld",
                (long long)MTL_CROSS_ENTROPY_MAX_ELEMENTS, (long long)B, (long long)C);
    mtl_launch_pdl(ctx, k_cross_entropy_fwd, dim3(1), dim3(kLossBlock), (size_t)(0), loss, (float*)nullptr, logits, y_true, (int)B, (int)C, scale);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_cross_entropy_fwd_grad(mtl_ctx* ctx, float* loss, float* dlogits, const float* logits, const float* y_true,
                                   int64_t B, int64_t C, float scale) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, loss && dlogits && logits && y_true, "null pointer in mtl_cross_entropy_fwd_grad");
    MTL_REQUIRE(ctx, B >= 1 && C >= 1 && B * C <= MTL_CROSS_ENTROPY_MAX_ELEMENTS,
                "mtl_cross_entropy_fwd_grad handles up to %lld logits, got %lld x %lld",
                (long long)MTL_CROSS_ENTROPY_MAX_ELEMENTS, (long long)B, (long long)C);
    const int grad_blocks = (int)((B + kLossBlock - 1) / kLossBlock);
    mtl_launch_pdl(ctx, k_cross_entropy_fwd, dim3(1 + grad_blocks), dim3(kLossBlock), (size_t)(0), loss, dlogits, logits, y_true, (int)B, (int)C, scale);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_cross_entropy_bwd(mtl_ctx* ctx, float* dlogits, const float* logits, const float* y_true, int64_t B,
                              int64_t C, float scale, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, dlogits && logits && y_true, "null pointer in mtl_cross_entropy_bwd");
    MTL_REQUIRE(ctx, B >= 1 && C >= 1 && B * C <= MTL_CROSS_ENTROPY_MAX_ELEMENTS,
                "mtl_cross_entropy_bwd handles up to %lld logits, got %lld x %lld",
                (long long)MTL_CROSS_ENTROPY_MAX_ELEMENTS, (long long)B, (long long)C);
    const int blocks = (int)((B + 255) / 256);
    mtl_launch_pdl(ctx, k_cross_entropy_bwd, dim3(blocks), dim3(256), (size_t)(0), dlogits, logits, y_true, (int)B, (int)C, scale, accumulate);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

}  // extern "C"
