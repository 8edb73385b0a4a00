// Fused Adam step over one flat fp32 arena: a single launch reads p, g, m, v and writes p, m, v
// (28 bytes per parameter), 128-bit accesses, grid sized to the SM count.
// Arithmetic order follows Adam.step, mantle/nn/optim.mojo:104-138.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int kBlock = 256;

struct AdamK {
    float lr, b1, b2, eps, omb1, omb2, c1, c2, gscale;
};

// beta ** iter with an integer exponent: exponentiation by squaring in fp32, the same on host and
// device.
__host__ __device__ __forceinline__ float pow_int(float b, int e) {
    float r = 1.0f;
    while (e > 0) {
        if (e & 1) r *= b;
        b *= b;
        e >>= 1;
    }
    return r;
}

__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const AdamK& k) {
    g *= k.gscale;
    m = k.b1 * m + k.omb1 * g;       // beta1 * momentum + (1 - beta1) * grad
    float mh = m / k.c1;             // / (1 - beta1 ** iter)
    v = k.b2 * v + k.omb2 * g * g;   // beta2 * rms + (1 - beta2) * grad * grad
    float vh = v / k.c2;             // / (1 - beta2 ** iter)
    p = p - k.lr * (mh / (sqrtf(vh) + k.eps));
}

__global__ void __launch_bounds__(kBlock) k_adam(float* __restrict__ p, const float* __restrict__ g,
                                                 float* __restrict__ m, float* __restrict__ v, int64_t n,
                                                 AdamK k, int vec, int32_t* __restrict__ t_dev,
                                                 int32_t* __restrict__ ticket) {
    mtl_pdl_sync();
    int t = 0;
    if (t_dev) {
        // the step count lives on the device (captured steps are replayed): this step is number *t_dev + 1
        t = *reinterpret_cast<volatile int32_t*>(t_dev) + 1;
        k.c1 = 1.0f - pow_int(k.b1, t);
        k.c2 = 1.0f - pow_int(k.b2, t);
    }
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    if (vec) {
        int64_t n4 = n >> 2;
        float4* p4 = reinterpret_cast<float4*>(p);
        const float4* g4 = reinterpret_cast<const float4*>(g);
        float4* m4 = reinterpret_cast<float4*>(m);
        float4* v4 = reinterpret_cast<float4*>(v);
        for (int64_t i = tid; i < n4; i += stride) {
            float4 pp = p4[i], gg = g4[i], mm = m4[i], vv = v4[i];
            adam_one(pp.x, gg.x, mm.x, vv.x, k);
            adam_one(pp.y, gg.y, mm.y, vv.y, k);
            adam_one(pp.z, gg.z, mm.z, vv.z, k);
            adam_one(pp.w, gg.w, mm.w, vv.w, k);
            p4[i] = pp; m4[i] = mm; v4[i] = vv;
        }
        for (int64_t i = (n4 << 2) + tid; i < n; i += stride) adam_one(p[i], g[i], m[i], v[i], k);
    } else {
        for (int64_t i = tid; i < n; i += stride) adam_one(p[i], g[i], m[i], v[i], k);
    }
    if (t_dev) {
        // every block has read the old count before it takes a ticket; the block that takes the last one
        // stores the new count and puts the ticket counter back
        __syncthreads();
        if (threadIdx.x == 0 && atomicAdd(ticket, 1) == (int)gridDim.x - 1) {
            *t_dev = t;
            *ticket = 0;
        }
    }
}

}  // namespace

static int32_t adam_launch(mtl_ctx* ctx, float* params, const float* grads, float* m, float* v, int64_t n,
                           float lr, float beta1, float beta2, float eps, int32_t t, float grad_scale,
                           int32_t* t_dev) {
    MTL_REQUIRE(ctx, n >= 0 && ((params && grads && m && v) || n == 0), "null pointer in mtl_adam_step");
    MTL_REQUIRE(ctx, t_dev || t >= 1, "Adam iteration count must be >= 1, got %d", t);
    AdamK k;
    k.lr = lr; k.b1 = beta1; k.b2 = beta2; k.eps = eps;
    k.omb1 = 1.0f - beta1;
    k.omb2 = 1.0f - beta2;
    // fp32 power of an fp32 base with the integer iteration count, `self.beta1**self.iter`
    k.c1 = 1.0f - pow_int(beta1, t_dev ? 1 : t);
    k.c2 = 1.0f - pow_int(beta2, t_dev ? 1 : t);
    k.gscale = grad_scale;
    int vec = ((((uintptr_t)params) | ((uintptr_t)grads) | ((uintptr_t)m) | ((uintptr_t)v)) & 15u) == 0;
    if (n == 0 && !t_dev) return MTL_OK;
    int grid = mtl_grid_for((n + 3) / 4, kBlock, ctx->sm_count, 8);
    mtl_launch_pdl(ctx, k_adam, dim3(grid), dim3(kBlock), (size_t)(0), params, grads, m, v, n, k, vec, t_dev, ctx->tickets + 8191);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

extern "C" {

int32_t mtl_adam_step(mtl_ctx* ctx, float* params, const float* grads, float* m, float* v, int64_t n, float lr,
                      float beta1, float beta2, float eps, int32_t t, float grad_scale) {
    MTL_CHECK_CTX(ctx);
    return adam_launch(ctx, params, grads, m, v, n, lr, beta1, beta2, eps, t, grad_scale, nullptr);
}

int32_t mtl_adam_step_dev(mtl_ctx* ctx, float* params, const float* grads, float* m, float* v, int64_t n,
                          float lr, float beta1, float beta2, float eps, int32_t* t_dev, float grad_scale) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, t_dev, "null iteration counter");
    return adam_launch(ctx, params, grads, m, v, n, lr, beta1, beta2, eps, 0, grad_scale, t_dev);
}

}  // extern "C"
