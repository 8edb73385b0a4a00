// CUDA-core CONV2D kernels: every padding / stride / dilation the reference accepts, and the
// layers whose GEMM view is too thin for the tensor cores (e.g. one input channel with a 5x5
// kernel: 25 multiply-adds per output, bound by writing the output).
//   forward      one thread per output element, weights staged in shared memory when they fit
//   input grad   gather form: one thread per input element, no atomics
//   kernel grad  per (out_ch, in_ch) block, taps accumulated in registers, deterministic
//                two-pass reduction over batch splits
//   bias grad    per out_ch block, two-pass
// Formulas: mantle/autograd/ops/conv.mojo:81-226 (forward), :284-338 (dX), :340-393 (dW),
// :395-423 (db).
#include "common.cuh"
#include "conv.cuh"

namespace {

constexpr int kBlock = 256;

__global__ void __launch_bounds__(kBlock) k_conv_fwd(float* __restrict__ Y, const float* __restrict__ X,
                                                     const float* __restrict__ Wt, const float* __restrict__ bias,
                                                     ConvGeom g, int64_t n_out, int w_in_smem) {
    extern __shared__ float w_s[];
    const int crs = g.C * g.R * g.S;
    if (w_in_smem) {
        for (int i = threadIdx.x; i < g.K * crs; i += blockDim.x) w_s[i] = Wt[i];
        __syncthreads();
    }
    const float* wsrc = w_in_smem ? w_s : Wt;
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int plane = g.OH * g.OW;
    for (int64_t o = tid; o < n_out; o += stride) {
        int64_t nk = o / plane;
        int rem = (int)(o - nk * plane);
        int oh = rem / g.OW, ow = rem - oh * g.OW;
        int n = (int)(nk / g.K), k = (int)(nk - (int64_t)n * g.K);
        const float* xn = X + (int64_t)n * g.C * g.H * g.W;
        const float* wk = wsrc + (int64_t)k * crs;
        int ih0 = oh * g.sh - g.ph, iw0 = ow * g.sw - g.pw;
        float acc = 0.0f;
        for (int c = 0; c < g.C; ++c) {
            const float* xc = xn + (int64_t)c * g.H * g.W;
            for (int r = 0; r < g.R; ++r) {
                int ih = ih0 + r * g.dh;
                if (ih < 0 || ih >= g.H) continue;
                for (int s = 0; s < g.S; ++s) {
                    int iw = iw0 + s * g.dw;
                    if (iw < 0 || iw >= g.W) continue;
                    acc = fmaf(__ldg(xc + ih * g.W + iw), wk[(c * g.R + r) * g.S + s], acc);
                }
            }
        }
        Y[o] = acc + (bias ? __ldg(bias + k) : 0.0f);
    }
}

// Forward for thin inputs (C*R*S <= 75, e.g. one input channel with a 5x5 kernel): one thread per
// output pixel keeps its input patch in registers and produces every output channel, reading the
// weights as 128-bit broadcasts from shared memory; stores of one channel are coalesced across the
// warp.  Bound by writing Y.
template <int R, int S, int C>
__global__ void __launch_bounds__(kBlock) k_conv_fwd_patch(float* __restrict__ Y, const float* __restrict__ X,
                                                           const float* __restrict__ Wt,
                                                           const float* __restrict__ bias, ConvGeom g, int64_t n_pix) {
    constexpr int CRS = C * R * S;
    constexpr int CRS4 = (CRS + 3) / 4 * 4;
    extern __shared__ float w_s[];  // [K][CRS4] zero padded, then bias[K]
    float* b_s = w_s + g.K * CRS4;
    for (int i = threadIdx.x; i < g.K * CRS4; i += blockDim.x) {
        int k = i / CRS4, j = i - k * CRS4;
        w_s[i] = j < CRS ? Wt[k * CRS + j] : 0.0f;
    }
    for (int i = threadIdx.x; i < g.K; i += blockDim.x) b_s[i] = bias ? bias[i] : 0.0f;
    __syncthreads();
    const int plane = g.OH * g.OW;
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t p = tid; p < n_pix; p += stride) {
        int n = (int)(p / plane);
        int rem = (int)(p - (int64_t)n * plane);
        int oh = rem / g.OW, ow = rem - oh * g.OW;
        int ih0 = oh * g.sh - g.ph, iw0 = ow * g.sw - g.pw;
        float patch[CRS4];
#pragma unroll
        for (int c = 0; c < C; ++c)
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int s2 = 0; s2 < S; ++s2) {
                    int ih = ih0 + r * g.dh, iw = iw0 + s2 * g.dw;
                    bool ok = ih >= 0 && ih < g.H && iw >= 0 && iw < g.W;
                    patch[(c * R + r) * S + s2] = ok ? __ldg(X + (((int64_t)n * C + c) * g.H + ih) * g.W + iw) : 0.0f;
                }
#pragma unroll
        for (int j = CRS; j < CRS4; ++j) patch[j] = 0.0f;
        float* yp = Y + (int64_t)n * g.K * plane + rem;
        for (int k = 0; k < g.K; ++k) {
            const float4* wk = reinterpret_cast<const float4*>(w_s + k * CRS4);
            float acc = 0.0f;
#pragma unroll
            for (int j = 0; j < CRS4 / 4; ++j) {
                float4 w = wk[j];
                acc = fmaf(patch[4 * j], w.x, acc);
                acc = fmaf(patch[4 * j + 1], w.y, acc);
                acc = fmaf(patch[4 * j + 2], w.z, acc);
                acc = fmaf(patch[4 * j + 3], w.w, acc);
            }
            yp[(int64_t)k * plane] = acc + b_s[k];
        }
    }
}

// Forward for few input channels and rows of at most 32 - (S - 1) pixels: a warp owns one output
// row, a lane one output channel with its R*S*C weights in registers.  Input rows come out of a
// zero-padded plane in shared memory as broadcast float4 loads (8*R*C loads for OW*R*S*C FMAs);
// the finished 32 channels x OW block is turned through shared memory so that OW/4 lanes store one
// channel's row as consecutive float4s.  Bound by writing Y.
// POOL: a warp produces two adjacent output rows, applies the activation and writes only their
// 2x2 / stride-2 maxima and argmax indices (MAXPOOL2D.forward's strict '>' scan in row-major window
// order, pool.mojo:44-100), so the full-size activation never reaches memory.
template <int R, int S, int C, int OW, int WARPS, bool POOL>
__global__ void __launch_bounds__(WARPS * 32, 2) k_conv_fwd_rows(float* __restrict__ Y, int32_t* __restrict__ pool_idx,
                                                                  float* __restrict__ pooled_cl,
                                                                  const float* __restrict__ X,
                                                                  const float* __restrict__ Wt,
                                                                  const float* __restrict__ bias, ConvGeom g, int relu) {
    constexpr int PW = 32, NT = WARPS * 32, SST = OW + ((OW / 4) % 2 == 0 ? 4 : 8);  // odd multiple of 4 floats
    constexpr int LPC = OW / 4, CPI = 32 / LPC;  // lanes per channel row, channel rows per store instruction
    extern __shared__ __align__(16) float rows_smem[];
    const int PH = g.OH + R - 1;
    float* xs = rows_smem;                         // [2][C][PH][PW]
    float* stg = rows_smem + 2 * C * PH * PW;      // [WARPS][32][SST]
    const int kgroups = (g.K + 31) / 32;
    const int kg = blockIdx.x % kgroups;
    const int k0 = kg * 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k = k0 + lane;
    float w[C * R * S];
#pragma unroll
    for (int i = 0; i < C * R * S; ++i) w[i] = k < g.K ? __ldg(Wt + (int64_t)k * C * R * S + i) : 0.0f;
    const float bv = (bias && k < g.K) ? __ldg(bias + k) : 0.0f;

    for (int i = threadIdx.x; i < 2 * C * PH * PW; i += NT) xs[i] = 0.0f;
    __syncthreads();
    const int n_first = blockIdx.x / kgroups, n_step = gridDim.x / kgroups;
    auto issue = [&](int n, int buf) {
        float* xb = xs + buf * C * PH * PW;
        const float* xn = X + (int64_t)n * C * g.H * g.W;
        for (int i = threadIdx.x; i < C * g.H * g.W; i += NT) {
            const int c = i / (g.H * g.W), rem = i - c * g.H * g.W;
            const int ih = rem / g.W, iw = rem - ih * g.W;
            uint32_t dst = (uint32_t)__cvta_generic_to_shared(xb + (c * PH + ih + g.ph) * PW + iw + g.pw);
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(xn + i) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (n_first < g.N) issue(n_first, 0);
    int buf = 0;
    float* sw = stg + warp * 32 * SST;
    const int chl = lane / LPC, sub = lane - chl * LPC;
    for (int n = n_first; n < g.N; n += n_step, buf ^= 1) {
        if (n + n_step < g.N) {
            issue(n + n_step, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* xb = xs + buf * C * PH * PW;
        auto row = [&](int oh, float (&out)[OW]) {
#pragma unroll
            for (int i = 0; i < OW; ++i) out[i] = bv;
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    float xr[PW];
#pragma unroll
                    for (int i = 0; i < PW / 4; ++i) {
                        const float4 q = *reinterpret_cast<const float4*>(xb + (c * PH + oh + r) * PW + 4 * i);
                        xr[4 * i] = q.x; xr[4 * i + 1] = q.y; xr[4 * i + 2] = q.z; xr[4 * i + 3] = q.w;
                    }
#pragma unroll
                    for (int ow = 0; ow < OW; ++ow)
#pragma unroll
                        for (int s2 = 0; s2 < S; ++s2) out[ow] = fmaf(w[(c * R + r) * S + s2], xr[ow + s2], out[ow]);
                }
            if (relu) {  // RELU.forward: x > 0 ? x : 0
#pragma unroll
                for (int i = 0; i < OW; ++i) out[i] = out[i] > 0.0f ? out[i] : 0.0f;
            }
        };
        if constexpr (!POOL) {
            for (int oh = warp; oh < g.OH; oh += WARPS) {
                float out[OW];
                row(oh, out);
                __syncwarp();
#pragma unroll
                for (int i = 0; i < OW / 4; ++i)
                    *reinterpret_cast<float4*>(sw + lane * SST + 4 * i) = make_float4(out[4 * i], out[4 * i + 1], out[4 * i + 2], out[4 * i + 3]);
                __syncwarp();
                if (chl < CPI) {
#pragma unroll
                    for (int it = 0; it < (32 + CPI - 1) / CPI; ++it) {
                        const int ch = it * CPI + chl;
                        if (ch < 32 && k0 + ch < g.K) {
                            const float4 q = *reinterpret_cast<const float4*>(sw + ch * SST + 4 * sub);
                            *reinterpret_cast<float4*>(Y + (((int64_t)n * g.K + k0 + ch) * g.OH + oh) * OW + 4 * sub) = q;
                        }
                    }
                }
            }
        } else {
            constexpr int POW = OW / 2, PST = POW + 1;   // odd row stride: conflict-free scalar access
            const int POH = g.OH / 2;
            int32_t* swi = reinterpret_cast<int32_t*>(sw + 32 * PST);
            for (int pr = warp; pr < POH; pr += WARPS) {
                float o0[OW], o1[OW];
                row(2 * pr, o0);
                row(2 * pr + 1, o1);
                __syncwarp();
#pragma unroll
                for (int pw = 0; pw < POW; ++pw) {
                    const int i00 = (2 * pr) * OW + 2 * pw;
                    float m = -INFINITY;
                    int j = -1;
                    if (o0[2 * pw] > m) { m = o0[2 * pw]; j = i00; }
                    if (o0[2 * pw + 1] > m) { m = o0[2 * pw + 1]; j = i00 + 1; }
                    if (o1[2 * pw] > m) { m = o1[2 * pw]; j = i00 + OW; }
                    if (o1[2 * pw + 1] > m) { m = o1[2 * pw + 1]; j = i00 + OW + 1; }
                    sw[lane * PST + pw] = m;
                    swi[lane * PST + pw] = j;
                    // channels-last twin [N, POH, POW, K] for the layer that reads this output: the
                    // lanes are adjacent channels, so this store is coalesced as it stands
                    if (pooled_cl && k < g.K) pooled_cl[(((int64_t)n * POH + pr) * POW + pw) * g.K + k] = m;
                }
                __syncwarp();
                for (int e = lane; e < 32 * POW; e += 32) {
                    const int ch = e / POW, pw = e - ch * POW;
                    if (k0 + ch < g.K) {
                        const int64_t o = (((int64_t)n * g.K + k0 + ch) * POH + pr) * POW + pw;
                        Y[o] = sw[ch * PST + pw];
                        if (pool_idx) pool_idx[o] = swi[ch * PST + pw];
                    }
                }
            }
        }
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kBlock) k_conv_dgrad(float* __restrict__ dX, const float* __restrict__ ug,
                                                       const float* __restrict__ Wt, ConvGeom g, int64_t n_in,
                                                       int accumulate) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const int plane = g.H * g.W;
    for (int64_t i = tid; i < n_in; i += stride) {
        int64_t nc = i / plane;
        int rem = (int)(i - nc * plane);
        int ih = rem / g.W, iw = rem - ih * g.W;
        int n = (int)(nc / g.C), c = (int)(nc - (int64_t)n * g.C);
        float acc = 0.0f;
        for (int r = 0; r < g.R; ++r) {
            int th = ih + g.ph - r * g.dh;
            if (th < 0 || th % g.sh) continue;
            int oh = th / g.sh;
            if (oh >= g.OH) continue;
            for (int s = 0; s < g.S; ++s) {
                int tw = iw + g.pw - s * g.dw;
                if (tw < 0 || tw % g.sw) continue;
                int ow = tw / g.sw;
                if (ow >= g.OW) continue;
                const float* up = ug + ((int64_t)n * g.K * g.OH + oh) * g.OW + ow;
                const float* wp = Wt + ((int64_t)c * g.R + r) * g.S + s;
                for (int k = 0; k < g.K; ++k)
                    acc = fmaf(__ldg(up + (int64_t)k * g.OH * g.OW), __ldg(wp + (int64_t)k * g.C * g.R * g.S), acc);
            }
        }
        dX[i] = accumulate ? dX[i] + acc : acc;
    }
}

__device__ __forceinline__ float block_sum(float v, float* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) smem[threadIdx.x >> 5] = v;
    __syncthreads();
    float t = 0.0f;
    if (threadIdx.x < 32) {
        t = threadIdx.x < (kBlock >> 5) ? smem[threadIdx.x] : 0.0f;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    }
    __syncthreads();
    return t;
}

// Kernel gradient, taps in registers.  grid = (K*C, nsplit); partial[split][kc][tap].
template <int R, int S>
__global__ void __launch_bounds__(kBlock) k_conv_wgrad_taps(float* __restrict__ partial, const float* __restrict__ ug,
                                                            const float* __restrict__ X, ConvGeom g, int n_per_split) {
    __shared__ float smem[32];
    const int kc = blockIdx.x;
    const int k = kc / g.C, c = kc - k * g.C;
    const int n_begin = blockIdx.y * n_per_split;
    const int n_end = min(g.N, n_begin + n_per_split);
    const int plane = g.OH * g.OW;
    float acc[R * S];
#pragma unroll
    for (int t = 0; t < R * S; ++t) acc[t] = 0.0f;
    const int64_t total = (int64_t)(n_end - n_begin) * plane;
    for (int64_t e = threadIdx.x; e < total; e += kBlock) {
        int n = n_begin + (int)(e / plane);
        int rem = (int)(e % plane);
        int oh = rem / g.OW, ow = rem - oh * g.OW;
        float u = __ldg(ug + ((int64_t)n * g.K + k) * plane + rem);
        const float* xc = X + ((int64_t)n * g.C + c) * g.H * g.W;
        int ih0 = oh * g.sh - g.ph, iw0 = ow * g.sw - g.pw;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            int ih = ih0 + r * g.dh;
            bool rok = ih >= 0 && ih < g.H;
#pragma unroll
            for (int s = 0; s < S; ++s) {
                int iw = iw0 + s * g.dw;
                float x = (rok && iw >= 0 && iw < g.W) ? __ldg(xc + ih * g.W + iw) : 0.0f;
                acc[r * S + s] = fmaf(x, u, acc[r * S + s]);
            }
        }
    }
    float* out = partial + ((int64_t)blockIdx.y * g.K * g.C + kc) * (R * S);
#pragma unroll
    for (int t = 0; t < R * S; ++t) {
        float v = block_sum(acc[t], smem);
        if (threadIdx.x == 0) out[t] = v;
    }
}

// Kernel gradient with the input plane staged in shared memory (zero halo included, so taps need
// no bounds checks) and KB output channels per block: per pixel R*S shared loads feed KB*R*S FMAs,
// and every element of ug is read exactly once.  grid = ((K/KB)*C, nsplit); partial[split][kc][tap].
template <int R, int S, int KB>
__global__ void __launch_bounds__(kBlock) k_conv_wgrad_staged(float* __restrict__ partial,
                                                              const float* __restrict__ ug,
                                                              const float* __restrict__ X, ConvGeom g,
                                                              int n_per_split, int PH, int PW) {
    extern __shared__ float x_s[];                 // [PH][PW] padded plane
    __shared__ float red[kBlock / 32][KB * R * S];
    const int kgroups = (g.K + KB - 1) / KB;
    const int kg = blockIdx.x % kgroups, c = blockIdx.x / kgroups;
    const int k0 = kg * KB;
    const int n_begin = blockIdx.y * n_per_split;
    const int n_end = min(g.N, n_begin + n_per_split);
    const int plane = g.OH * g.OW;
    float acc[KB][R * S];
#pragma unroll
    for (int a = 0; a < KB; ++a)
#pragma unroll
        for (int t = 0; t < R * S; ++t) acc[a][t] = 0.0f;
    for (int n = n_begin; n < n_end; ++n) {
        const float* xc = X + ((int64_t)n * g.C + c) * g.H * g.W;
        __syncthreads();
        for (int i = threadIdx.x; i < PH * PW; i += kBlock) {
            int ih = i / PW - g.ph, iw = i % PW - g.pw;
            x_s[i] = (ih >= 0 && ih < g.H && iw >= 0 && iw < g.W) ? __ldg(xc + ih * g.W + iw) : 0.0f;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < plane; e += kBlock) {
            int oh = e / g.OW, ow = e - oh * g.OW;
            float u[KB];
#pragma unroll
            for (int a = 0; a < KB; ++a)
                u[a] = (k0 + a < g.K) ? __ldg(ug + ((int64_t)n * g.K + k0 + a) * plane + e) : 0.0f;
            const float* xp = x_s + (oh * g.sh) * PW + ow * g.sw;
#pragma unroll
            for (int r = 0; r < R; ++r)
#pragma unroll
                for (int s2 = 0; s2 < S; ++s2) {
                    float x = xp[r * g.dh * PW + s2 * g.dw];
#pragma unroll
                    for (int a = 0; a < KB; ++a) acc[a][r * S + s2] = fmaf(x, u[a], acc[a][r * S + s2]);
                }
        }
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
    for (int a = 0; a < KB; ++a)
#pragma unroll
        for (int t = 0; t < R * S; ++t) {
            float v = acc[a][t];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) red[warp][a * R * S + t] = v;
        }
    __syncthreads();
    for (int i = threadIdx.x; i < KB * R * S; i += kBlock) {
        int a = i / (R * S), t = i - a * (R * S);
        if (k0 + a >= g.K) continue;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < kBlock / 32; ++w) v += red[w][i];
        partial[((int64_t)blockIdx.y * g.K * g.C + (int64_t)(k0 + a) * g.C + c) * (R * S) + t] = v;
    }
}

// Few input channels, stride 1, rows of at most 32 - (S - 1) pixels (the first layer of the CNNs).
// This layer is bound by reading ug once, so ug streams through shared memory with cp.async
// (two buffers) while the previous chunk is multiplied.  A warp owns one output row, a lane one
// output channel: the input row comes out of shared memory as broadcast float4 loads and the ug
// row as one float4 per four pixels (row stride 4 mod 32 floats keeps those conflict free), so
// one output row costs 8*R + OW/4 shared loads for OW*R*S FMAs per thread.
template <int R, int S, int OW, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 3) k_conv_wgrad_rows(float* __restrict__ partial,
                                                                const float* __restrict__ ug,
                                                                const float* __restrict__ X, ConvGeom g,
                                                                int n_per_split, int ustride,
                                                                float* __restrict__ bias_partial) {
    constexpr int PW = 32, RS = R * S, NT = WARPS * 32;
    extern __shared__ __align__(16) float rows_smem[];
    const int PH = g.OH + R - 1;
    float* xs = rows_smem;                       // [2][PH][PW] zero-padded input planes
    float* us = rows_smem + 2 * PH * PW;         // [2][32][ustride] chunks of ug
    const int kgroups = (g.K + 31) / 32;
    const int kg = blockIdx.x % kgroups, c = blockIdx.x / kgroups;
    const int k0 = kg * 32;
    const int n_begin = blockIdx.y * n_per_split;
    const int n_end = min(g.N, n_begin + n_per_split);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nchunks = (g.OH + WARPS - 1) / WARPS;
    const int steps = (n_end - n_begin) * nchunks;

    for (int i = threadIdx.x; i < 2 * PH * PW; i += NT) xs[i] = 0.0f;
    __syncthreads();

    auto issue = [&](int step) {
        const int n = n_begin + step / nchunks, chunk = step % nchunks;
        const int oh0 = chunk * WARPS;
        constexpr int pieces = WARPS * OW / 4;  // 16-byte pieces per channel (OH is a multiple of WARPS)
        float* ub = us + (step & 1) * 32 * ustride;
        const float* ubase = ug + (((int64_t)n * g.K + k0) * g.OH + oh0) * OW;
        const int plane = g.OH * OW;
#pragma unroll
        for (int i = threadIdx.x; i < 32 * pieces; i += NT) {
            const int kk = i / pieces, pc = i - kk * pieces;
            if (k0 + kk < g.K) {
                const float* src = ubase + kk * plane + pc * 4;
                uint32_t dst = (uint32_t)__cvta_generic_to_shared(ub + kk * ustride + pc * 4);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
            }
        }
        if (chunk == 0) {
            float* xb = xs + ((step / nchunks) & 1) * PH * PW;
            const float* xc = X + ((int64_t)n * g.C + c) * g.H * g.W;
            for (int i = threadIdx.x; i < g.H * g.W; i += NT) {
                const int ih = i / g.W, iw = i - ih * g.W;
                uint32_t dst = (uint32_t)__cvta_generic_to_shared(xb + (ih + g.ph) * PW + iw + g.pw);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(xc + i) : "memory");
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[RS];
#pragma unroll
    for (int t = 0; t < RS; ++t) acc[t] = 0.0f;
    float bsum = 0.0f;  // sum of this lane's channel over the rows this warp sees (bias gradient)

    if (steps > 0) issue(0);
    for (int step = 0; step < steps; ++step) {
        if (step + 1 < steps) {
            issue(step + 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const int chunk = step % nchunks;
        const int oh = chunk * WARPS + warp;
        if (oh < g.OH) {
            const float* ub = us + (step & 1) * 32 * ustride + lane * ustride + warp * OW;
            const float* xb = xs + ((step / nchunks) & 1) * PH * PW + oh * PW;
            float u[OW];
#pragma unroll
            for (int i = 0; i < OW / 4; ++i) {
                const float4 q = *reinterpret_cast<const float4*>(ub + 4 * i);
                u[4 * i] = q.x; u[4 * i + 1] = q.y; u[4 * i + 2] = q.z; u[4 * i + 3] = q.w;
                bsum += (q.x + q.y) + (q.z + q.w);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float xr[PW];
#pragma unroll
                for (int i = 0; i < PW / 4; ++i) {
                    const float4 q = *reinterpret_cast<const float4*>(xb + r * PW + 4 * i);
                    xr[4 * i] = q.x; xr[4 * i + 1] = q.y; xr[4 * i + 2] = q.z; xr[4 * i + 3] = q.w;
                }
#pragma unroll
                for (int ow = 0; ow < OW; ++ow)
#pragma unroll
                    for (int s2 = 0; s2 < S; ++s2) acc[r * S + s2] = fmaf(u[ow], xr[ow + s2], acc[r * S + s2]);
            }
        }
        __syncthreads();
    }
    // fold the WARPS row partials of every channel in a fixed order
    float* red = us;  // [WARPS][32][RS]
#pragma unroll
    for (int t = 0; t < RS; ++t) red[(warp * 32 + lane) * RS + t] = acc[t];
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * RS; i += NT) {
        const int kk = i / RS, t = i - kk * RS;
        if (k0 + kk >= g.K) continue;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[w * 32 * RS + i];
        partial[((int64_t)blockIdx.y * g.K * g.C + (int64_t)(k0 + kk) * g.C + c) * RS + t] = v;
    }
    if (bias_partial && c == 0) {  // every input channel sees the same ug: one of them reports
        __syncthreads();
        red[warp * 32 + lane] = bsum;
        __syncthreads();
        if (threadIdx.x < 32 && k0 + threadIdx.x < g.K) {
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += red[w * 32 + threadIdx.x];
            bias_partial[(int64_t)blockIdx.y * g.K + k0 + threadIdx.x] = v;
        }
    }
}

// The same kernel gradient for a layer followed by RELU and a 2x2 / stride-2 MAXPOOL2D, fed with the
// POOLED upper gradient: pg (gradient of the pooling output), pidx (argmax indices of the forward
// pass) and pv (pooled values, the RELU mask of the selected element).  The dense gradient of the
// layer's output -- zero except one element per window -- is rebuilt 14 rows at a time in shared
// memory (every thread writes the 2x2 windows of 14 pooled elements, so nothing has to be cleared)
// and never exists in global memory.  The pooled data of the next chunk are fetched into registers
// while the current chunk is multiplied.
template <int R, int S, int OW, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 2) k_conv_wgrad_rows_pooled(float* __restrict__ partial,
                                                                          const float* __restrict__ pg,
                                                                          const int32_t* __restrict__ pidx,
                                                                          const float* __restrict__ pv,
                                                                          const float* __restrict__ X, ConvGeom g,
                                                                          int n_per_split, int relu,
                                                                          float* __restrict__ bias_partial) {
    constexpr int PW = 32, RS = R * S, NT = WARPS * 32;
    constexpr int CR = 2 * WARPS;            // dense rows per chunk
    constexpr int POW = OW / 2, PRC = WARPS; // pooled row length, pooled rows per chunk
    constexpr int EPT = POW;                 // pooled elements per thread and chunk: 32 * PRC * POW / NT
    constexpr int UST = CR * OW + (((CR * OW) / 4) % 2 == 0 ? 4 : 0);  // odd multiple of 4 floats
    extern __shared__ __align__(16) float rows_smem[];
    const int PH = g.OH + R - 1;
    float* xs = rows_smem;                   // [2][PH][PW] zero-padded input planes
    float* tile = rows_smem + 2 * PH * PW;   // [32][UST] dense gradient rows of one chunk
    const int kgroups = (g.K + 31) / 32;
    const int kg = blockIdx.x % kgroups, c = blockIdx.x / kgroups;
    const int k0 = kg * 32;
    const int n_begin = blockIdx.y * n_per_split;
    const int n_end = min(g.N, n_begin + n_per_split);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nchunks = g.OH / CR;
    const int POH = g.OH / 2;
    const int steps = (n_end - n_begin) * nchunks;

    for (int i = threadIdx.x; i < 2 * PH * PW; i += NT) xs[i] = 0.0f;
    __syncthreads();

    // thread tid owns pooled row (channel tid / PRC, pooled row tid % PRC) of every chunk: POW
    // consecutive elements in global memory, two dense rows of OW consecutive floats in the tile
    float pgr[EPT];
    int pir[EPT];
    const int my_kk = threadIdx.x / PRC, my_phl = threadIdx.x - my_kk * PRC;
    const bool my_valid = k0 + my_kk < g.K;
    auto fetch = [&](int step) {  // pooled data of chunk `step` into registers, input plane of a new image
        const int n = n_begin + step / nchunks, chunk = step % nchunks;
        const int64_t o = (((int64_t)n * g.K + k0 + my_kk) * POH + chunk * PRC + my_phl) * POW;
#pragma unroll
        for (int j = 0; j < EPT; j += 2) {
            float2 v = make_float2(0.0f, 0.0f);
            int2 id = make_int2(-1, -1);
            if (my_valid) {
                v = __ldg(reinterpret_cast<const float2*>(pg + o + j));
                id = __ldg(reinterpret_cast<const int2*>(pidx + o + j));
                if (relu) {  // RELU.backward on the selected element
                    const float2 y = __ldg(reinterpret_cast<const float2*>(pv + o + j));
                    v.x = (y.x > 0.0f ? 1.0f : 0.0f) * v.x;
                    v.y = (y.y > 0.0f ? 1.0f : 0.0f) * v.y;
                }
            }
            pgr[j] = v.x; pgr[j + 1] = v.y;
            pir[j] = id.x; pir[j + 1] = id.y;
        }
        if (chunk == 0) {
            float* xb = xs + ((step / nchunks) & 1) * PH * PW;
            const float* xc = X + ((int64_t)n * g.C + c) * g.H * g.W;
            for (int i = threadIdx.x; i < g.H * g.W; i += NT) {
                const int ih = i / g.W, iw = i - ih * g.W;
                uint32_t dst = (uint32_t)__cvta_generic_to_shared(xb + (ih + g.ph) * PW + iw + g.pw);
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(xc + i) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
    };
    auto scatter = [&](int step) {  // MAXPOOL2D.backward of the fetched elements into the tile
        const int chunk = step % nchunks;
        const int i00 = (chunk * CR + 2 * my_phl) * OW;  // plane-local index of this thread's first window
        float* dst = tile + my_kk * UST + (2 * my_phl) * OW;
#pragma unroll
        for (int j = 0; j < EPT; j += 2) {
            // d = 0, 1, OW, OW + 1 inside the window, anything else (no argmax) leaves zeros
            const int d0 = pir[j] - (i00 + 2 * j), d1 = pir[j + 1] - (i00 + 2 * j + 2);
            const float v0 = pgr[j], v1 = pgr[j + 1];
            *reinterpret_cast<float4*>(dst + 2 * j) =
                make_float4(d0 == 0 ? v0 : 0.0f, d0 == 1 ? v0 : 0.0f, d1 == 0 ? v1 : 0.0f, d1 == 1 ? v1 : 0.0f);
            *reinterpret_cast<float4*>(dst + OW + 2 * j) =
                make_float4(d0 == OW ? v0 : 0.0f, d0 == OW + 1 ? v0 : 0.0f, d1 == OW ? v1 : 0.0f, d1 == OW + 1 ? v1 : 0.0f);
        }
    };

    float acc[RS];
#pragma unroll
    for (int t = 0; t < RS; ++t) acc[t] = 0.0f;
    float bsum = 0.0f;

    if (steps > 0) {
        fetch(0);
        scatter(0);
    }
    for (int step = 0; step < steps; ++step) {
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();  // tile of this chunk complete, input plane of this image landed
        if (step + 1 < steps) fetch(step + 1);  // in flight while this chunk is multiplied
        const int chunk = step % nchunks;
        const float* xplane = xs + ((step / nchunks) & 1) * PH * PW;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
            const int lr = 2 * warp + half;
            const int oh = chunk * CR + lr;
            const float* ub = tile + lane * UST + lr * OW;
            const float* xb = xplane + oh * PW;
            float u[OW];
#pragma unroll
            for (int i = 0; i < OW / 4; ++i) {
                const float4 q = *reinterpret_cast<const float4*>(ub + 4 * i);
                u[4 * i] = q.x; u[4 * i + 1] = q.y; u[4 * i + 2] = q.z; u[4 * i + 3] = q.w;
                bsum += (q.x + q.y) + (q.z + q.w);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                float xr[PW];
#pragma unroll
                for (int i = 0; i < PW / 4; ++i) {
                    const float4 q = *reinterpret_cast<const float4*>(xb + r * PW + 4 * i);
                    xr[4 * i] = q.x; xr[4 * i + 1] = q.y; xr[4 * i + 2] = q.z; xr[4 * i + 3] = q.w;
                }
#pragma unroll
                for (int ow = 0; ow < OW; ++ow)
#pragma unroll
                    for (int s2 = 0; s2 < S; ++s2) acc[r * S + s2] = fmaf(u[ow], xr[ow + s2], acc[r * S + s2]);
            }
        }
        __syncthreads();
        if (step + 1 < steps) scatter(step + 1);
    }
    __syncthreads();
    float* red = tile;  // [WARPS][32][RS]
#pragma unroll
    for (int t = 0; t < RS; ++t) red[(warp * 32 + lane) * RS + t] = acc[t];
    __syncthreads();
    for (int i = threadIdx.x; i < 32 * RS; i += NT) {
        const int kk = i / RS, t = i - kk * RS;
        if (k0 + kk >= g.K) continue;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) v += red[w * 32 * RS + i];
        partial[((int64_t)blockIdx.y * g.K * g.C + (int64_t)(k0 + kk) * g.C + c) * RS + t] = v;
    }
    if (bias_partial && c == 0) {
        __syncthreads();
        red[warp * 32 + lane] = bsum;
        __syncthreads();
        if (threadIdx.x < 32 && k0 + threadIdx.x < g.K) {
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < WARPS; ++w) v += red[w * 32 + threadIdx.x];
            bias_partial[(int64_t)blockIdx.y * g.K + k0 + threadIdx.x] = v;
        }
    }
}

// Any kernel size: one tap at a time.
__global__ void __launch_bounds__(kBlock) k_conv_wgrad_generic(float* __restrict__ partial, const float* __restrict__ ug,
                                                               const float* __restrict__ X, ConvGeom g,
                                                               int n_per_split) {
    __shared__ float smem[32];
    const int kc = blockIdx.x;
    const int k = kc / g.C, c = kc - k * g.C;
    const int n_begin = blockIdx.y * n_per_split;
    const int n_end = min(g.N, n_begin + n_per_split);
    const int plane = g.OH * g.OW;
    const int64_t total = (int64_t)(n_end - n_begin) * plane;
    float* out = partial + ((int64_t)blockIdx.y * g.K * g.C + kc) * (g.R * g.S);
    for (int r = 0; r < g.R; ++r)
        for (int s = 0; s < g.S; ++s) {
            float acc = 0.0f;
            for (int64_t e = threadIdx.x; e < total; e += kBlock) {
                int n = n_begin + (int)(e / plane);
                int rem = (int)(e % plane);
                int oh = rem / g.OW, ow = rem - oh * g.OW;
                int ih = oh * g.sh - g.ph + r * g.dh, iw = ow * g.sw - g.pw + s * g.dw;
                if (ih < 0 || ih >= g.H || iw < 0 || iw >= g.W) continue;
                acc = fmaf(__ldg(X + (((int64_t)n * g.C + c) * g.H + ih) * g.W + iw),
                           __ldg(ug + ((int64_t)n * g.K + k) * plane + rem), acc);
            }
            float v = block_sum(acc, smem);
            if (threadIdx.x == 0) out[r * g.S + s] = v;
        }
}

// grid = (K, nsplit); partial[split][k]
__global__ void __launch_bounds__(kBlock) k_conv_bgrad(float* __restrict__ partial, const float* __restrict__ ug,
                                                       int N, int K, int plane, int n_per_split) {
    __shared__ float smem[32];
    const int k = blockIdx.x;
    const int n_begin = blockIdx.y * n_per_split;
    const int n_end = min(N, n_begin + n_per_split);
    float acc = 0.0f;
    const bool vec = (plane % 4 == 0) && ((reinterpret_cast<uintptr_t>(ug) & 15u) == 0);
    if (vec) {
        // one flat index over (image, float4) keeps every thread busy with independent loads
        const int p4n = plane / 4;
        const int total = (n_end - n_begin) * p4n;
#pragma unroll 4
        for (int i = threadIdx.x; i < total; i += kBlock) {
            int n = n_begin + i / p4n, j = i - (i / p4n) * p4n;
            float4 v = __ldg(reinterpret_cast<const float4*>(ug + ((int64_t)n * K + k) * plane) + j);
            acc += (v.x + v.y) + (v.z + v.w);
        }
    } else {
        for (int n = n_begin; n < n_end; ++n) {
            const float* p = ug + ((int64_t)n * K + k) * plane;
            for (int i = threadIdx.x; i < plane; i += kBlock) acc += __ldg(p + i);
        }
    }
    float v = block_sum(acc, smem);
    if (threadIdx.x == 0) partial[(int64_t)blockIdx.y * K + k] = v;
}

}  // namespace

// out[i] (+)= sum over splits of partial[s][i]
__global__ void __launch_bounds__(256) k_sum_partials(float* __restrict__ out, const float* __restrict__ partial,
                                                      int64_t n, int nsplit, int accumulate) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) {
        float s = 0.0f;
        for (int j = 0; j < nsplit; ++j) s += partial[(int64_t)j * n + i];
        out[i] = accumulate ? out[i] + s : s;
    }
}

int32_t mtl_sum_partials(mtl_ctx* ctx, float* out, const float* partial, int64_t n, int nsplit, int accumulate) {
    int grid = mtl_grid_for(n, 256, ctx->sm_count, 8);
    k_sum_partials<<<grid, 256, 0, ctx->stream>>>(out, partial, n, nsplit, accumulate);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

template <int R, int S, int C>
static int32_t launch_fwd_patch(mtl_ctx* ctx, float* Y, const float* X, const float* Wt, const float* bias,
                                const ConvGeom& g) {
    constexpr int CRS4 = (C * R * S + 3) / 4 * 4;
    int64_t n_pix = (int64_t)g.N * g.OH * g.OW;
    size_t smem = ((size_t)g.K * CRS4 + g.K) * 4;
    int grid = mtl_grid_for(n_pix, kBlock, ctx->sm_count, 4);
    k_conv_fwd_patch<R, S, C><<<grid, kBlock, smem, ctx->stream>>>(Y, X, Wt, bias, g, n_pix);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

template <int R, int S, int C, bool POOL>
static int32_t launch_fwd_rows(mtl_ctx* ctx, float* Y, int32_t* pool_idx, float* pooled_cl, const float* X,
                               const float* Wt, const float* bias, const ConvGeom& g, int relu) {
    constexpr int WARPS = 7, OWc = 28, SST = 36;
    const int kgroups = (g.K + 31) / 32;
    const int PH = g.OH + R - 1;
    size_t smem = (size_t)(2 * C * PH * 32 + WARPS * 32 * SST) * 4;
    int per_group = (ctx->sm_count * 2 + kgroups - 1) / kgroups;
    if (per_group > g.N) per_group = g.N;
    auto kern = k_conv_fwd_rows<R, S, C, OWc, WARPS, POOL>;
    MTL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<per_group * kgroups, WARPS * 32, smem, ctx->stream>>>(Y, pool_idx, pooled_cl, X, Wt, bias, g, relu);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

static int32_t conv_fwd_simt_plain(mtl_ctx* ctx, float* Y, const float* X, const float* Wt, const float* bias,
                          const ConvGeom& g) {
    if ((size_t)g.K * (g.C * g.R * g.S + 4) * 4 <= 40 * 1024 && (int64_t)g.N * g.OH * g.OW >= 4096) {
        if (g.R == 5 && g.S == 5 && g.C == 1) return launch_fwd_patch<5, 5, 1>(ctx, Y, X, Wt, bias, g);
        if (g.R == 3 && g.S == 3 && g.C == 1) return launch_fwd_patch<3, 3, 1>(ctx, Y, X, Wt, bias, g);
        if (g.R == 3 && g.S == 3 && g.C == 3) return launch_fwd_patch<3, 3, 3>(ctx, Y, X, Wt, bias, g);
    }
    int64_t n_out = (int64_t)g.N * g.K * g.OH * g.OW;
    size_t wbytes = (size_t)g.K * g.C * g.R * g.S * 4;
    int w_in_smem = wbytes <= 40 * 1024;
    int grid = mtl_grid_for(n_out, kBlock, ctx->sm_count, 8);
    k_conv_fwd<<<grid, kBlock, w_in_smem ? wbytes : 0, ctx->stream>>>(Y, X, Wt, bias, g, n_out, w_in_smem);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

static bool fwd_rows_ok(const ConvGeom& g, const float* Y) {
    return g.OW == 28 && g.K >= 16 && g.sh == 1 && g.sw == 1 && g.dh == 1 && g.dw == 1 &&
           g.W + 2 * g.pw == g.OW + g.S - 1 && g.H + 2 * g.ph == g.OH + g.R - 1 && g.OH <= 64 &&
           ((reinterpret_cast<uintptr_t>(Y) & 15) == 0) && g.N >= 64 &&
           ((g.R == 5 && g.S == 5 && g.C == 1) || (g.R == 3 && g.S == 3 && (g.C == 1 || g.C == 3)));
}

int32_t mtl_conv_fwd_simt(mtl_ctx* ctx, float* Y, const float* X, const float* Wt, const float* bias,
                          const ConvGeom& g, int relu) {
    if (fwd_rows_ok(g, Y)) {
        if (g.R == 5) return launch_fwd_rows<5, 5, 1, false>(ctx, Y, nullptr, nullptr, X, Wt, bias, g, relu);
        if (g.C == 1) return launch_fwd_rows<3, 3, 1, false>(ctx, Y, nullptr, nullptr, X, Wt, bias, g, relu);
        return launch_fwd_rows<3, 3, 3, false>(ctx, Y, nullptr, nullptr, X, Wt, bias, g, relu);
    }
    int32_t rc = conv_fwd_simt_plain(ctx, Y, X, Wt, bias, g);
    if (rc || !relu) return rc;
    return mtl_unary_fwd(ctx, MTL_OP_RELU, Y, Y, (int64_t)g.N * g.K * g.OH * g.OW, 0.0f, 0.0f);
}

// CONV2D (+ RELU) followed by a 2x2 / stride-2 MAXPOOL2D in one kernel; false when this geometry has none.
bool mtl_conv_fwd_pool_simt_supported(const ConvGeom& g, const float* pooled) {
    return fwd_rows_ok(g, pooled) && g.OH % 2 == 0;
}

int32_t mtl_conv_fwd_pool_simt(mtl_ctx* ctx, float* pooled, int32_t* idx, float* pooled_cl, const float* X,
                               const float* Wt, const float* bias, const ConvGeom& g, int relu) {
    if (g.R == 5) return launch_fwd_rows<5, 5, 1, true>(ctx, pooled, idx, pooled_cl, X, Wt, bias, g, relu);
    if (g.C == 1) return launch_fwd_rows<3, 3, 1, true>(ctx, pooled, idx, pooled_cl, X, Wt, bias, g, relu);
    return launch_fwd_rows<3, 3, 3, true>(ctx, pooled, idx, pooled_cl, X, Wt, bias, g, relu);
}

int32_t mtl_conv_dgrad_simt(mtl_ctx* ctx, float* dX, const float* ug, const float* Wt, const ConvGeom& g,
                            int accumulate) {
    int64_t n_in = (int64_t)g.N * g.C * g.H * g.W;
    int grid = mtl_grid_for(n_in, kBlock, ctx->sm_count, 8);
    k_conv_dgrad<<<grid, kBlock, 0, ctx->stream>>>(dX, ug, Wt, g, n_in, accumulate);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

static int pick_nsplit(const mtl_ctx* ctx, int blocks_x, int N) {
    // enough blocks to fill the machine about four times over, never more splits than samples
    int want = (ctx->sm_count * 4 + blocks_x - 1) / blocks_x;
    if (want < 1) want = 1;
    if (want > N) want = N;
    if (want > 64) want = 64;
    return want;
}

// row-streaming variant: few input channels, 28-pixel rows, 'same'-style geometry
bool mtl_conv_wgrad_rows_supported(const ConvGeom& g, const float* ug) {
    return g.C <= 4 && g.K >= 16 && g.OW == 28 && g.OH % 7 == 0 && g.sh == 1 && g.sw == 1 && g.dh == 1 && g.dw == 1 &&
           ((g.R == 5 && g.S == 5) || (g.R == 3 && g.S == 3)) && g.W + 2 * g.pw == g.OW + g.S - 1 &&
           g.H + 2 * g.ph == g.OH + g.R - 1 && ((reinterpret_cast<uintptr_t>(ug) & 15) == 0) && g.N >= 64;
}

int32_t mtl_conv_wgrad_bias_rows(mtl_ctx* ctx, float* dW, float* db, const float* ug, const float* X, const ConvGeom& g,
                                 int acc_dw, int acc_db) {
    constexpr int WARPS = 7, OWc = 28;
    const int kc = g.K * g.C;
    const int taps = g.R * g.S;
    const int kgroups = (g.K + 31) / 32;
    int ustride = WARPS * OWc;
    while ((ustride / 4) % 2 == 0) ustride += 4;     // odd multiple of 4 floats
    const int PH = g.OH + g.R - 1;
    size_t smem = (size_t)(2 * PH * 32 + 2 * 32 * ustride) * 4;
    size_t red_bytes = (size_t)WARPS * 32 * taps * 4;
    if (red_bytes > (size_t)2 * 32 * ustride * 4) smem += red_bytes - (size_t)2 * 32 * ustride * 4;
    int ns = (ctx->sm_count * 3 + kgroups * g.C - 1) / (kgroups * g.C);
    if (ns > g.N / 4) ns = g.N / 4;
    if (ns < 1) ns = 1;
    int nps = (g.N + ns - 1) / ns;
    ns = (g.N + nps - 1) / nps;
    MTL_REQUIRE(ctx, ns <= 65535, "too many batch splits");
    void* ws2;
    int32_t rc2 = mtl_workspace(ctx, ((size_t)ns * kc * taps + (size_t)ns * g.K) * 4, &ws2);
    if (rc2) return rc2;
    float* part = (float*)ws2;
    float* bpart = db ? part + (size_t)ns * kc * taps : nullptr;
    dim3 rgrid((unsigned)(kgroups * g.C), (unsigned)ns);
    if (g.R == 5) {
        MTL_CUDA(ctx, cudaFuncSetAttribute(k_conv_wgrad_rows<5, 5, OWc, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k_conv_wgrad_rows<5, 5, OWc, WARPS><<<rgrid, WARPS * 32, smem, ctx->stream>>>(part, ug, X, g, nps, ustride, bpart);
    } else {
        MTL_CUDA(ctx, cudaFuncSetAttribute(k_conv_wgrad_rows<3, 3, OWc, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k_conv_wgrad_rows<3, 3, OWc, WARPS><<<rgrid, WARPS * 32, smem, ctx->stream>>>(part, ug, X, g, nps, ustride, bpart);
    }
    MTL_LAUNCHED(ctx);
    int32_t rc = mtl_sum_partials(ctx, dW, part, (int64_t)kc * taps, ns, acc_dw);
    if (rc || !db) return rc;
    return mtl_sum_partials(ctx, db, bpart, g.K, ns, acc_db);
}

// The pooled form of the row-streaming kernel gradient (see k_conv_wgrad_rows_pooled).
bool mtl_conv_wgrad_rows_pooled_supported(const ConvGeom& g) {
    return g.C <= 4 && g.K >= 16 && g.OW == 28 && g.OH % 14 == 0 && g.sh == 1 && g.sw == 1 && g.dh == 1 && g.dw == 1 &&
           ((g.R == 5 && g.S == 5) || (g.R == 3 && g.S == 3)) && g.W + 2 * g.pw == g.OW + g.S - 1 &&
           g.H + 2 * g.ph == g.OH + g.R - 1 && g.N >= 64;
}

int32_t mtl_conv_wgrad_bias_rows_pooled(mtl_ctx* ctx, float* dW, float* db, const float* pg, const int32_t* pidx,
                                        const float* pv, const float* X, const ConvGeom& g, int relu, int acc_dw,
                                        int acc_db) {
    constexpr int WARPS = 7, OWc = 28;
    const int kc = g.K * g.C;
    const int taps = g.R * g.S;
    const int kgroups = (g.K + 31) / 32;
    const int ust = 2 * WARPS * OWc + ((((2 * WARPS * OWc) / 4) % 2 == 0) ? 4 : 0);
    const int PH = g.OH + g.R - 1;
    size_t smem = (size_t)(2 * PH * 32 + 32 * ust) * 4;
    int ns = (ctx->sm_count * 2 + kgroups * g.C - 1) / (kgroups * g.C);
    if (ns > g.N / 4) ns = g.N / 4;
    if (ns < 1) ns = 1;
    int nps = (g.N + ns - 1) / ns;
    ns = (g.N + nps - 1) / nps;
    MTL_REQUIRE(ctx, ns <= 65535, "too many batch splits");
    void* ws2;
    int32_t rc2 = mtl_workspace(ctx, ((size_t)ns * kc * taps + (size_t)ns * g.K) * 4, &ws2);
    if (rc2) return rc2;
    float* part = (float*)ws2;
    float* bpart = db ? part + (size_t)ns * kc * taps : nullptr;
    dim3 rgrid((unsigned)(kgroups * g.C), (unsigned)ns);
    if (g.R == 5) {
        MTL_CUDA(ctx, cudaFuncSetAttribute(k_conv_wgrad_rows_pooled<5, 5, OWc, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k_conv_wgrad_rows_pooled<5, 5, OWc, WARPS><<<rgrid, WARPS * 32, smem, ctx->stream>>>(part, pg, pidx, pv, X, g, nps, relu, bpart);
    } else {
        MTL_CUDA(ctx, cudaFuncSetAttribute(k_conv_wgrad_rows_pooled<3, 3, OWc, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        k_conv_wgrad_rows_pooled<3, 3, OWc, WARPS><<<rgrid, WARPS * 32, smem, ctx->stream>>>(part, pg, pidx, pv, X, g, nps, relu, bpart);
    }
    MTL_LAUNCHED(ctx);
    if (dW) {
        int32_t rc = mtl_sum_partials(ctx, dW, part, (int64_t)kc * taps, ns, acc_dw);
        if (rc) return rc;
    }
    if (db) return mtl_sum_partials(ctx, db, bpart, g.K, ns, acc_db);
    return MTL_OK;
}

int32_t mtl_conv_wgrad_simt(mtl_ctx* ctx, float* dW, const float* ug, const float* X, const ConvGeom& g,
                            int accumulate) {
    const int kc = g.K * g.C;
    const int taps = g.R * g.S;
    int nsplit = pick_nsplit(ctx, kc, g.N);
    int n_per_split = (g.N + nsplit - 1) / nsplit;
    nsplit = (g.N + n_per_split - 1) / n_per_split;
    void* ws;
    int32_t rc = mtl_workspace(ctx, (size_t)nsplit * kc * taps * 4, &ws);
    if (rc) return rc;
    float* partial = (float*)ws;
    MTL_REQUIRE(ctx, nsplit <= 65535, "too many batch splits");
    // staged variant: padded input plane in shared memory, 4 output channels per block
    const int PH = (g.OH - 1) * g.sh + (g.R - 1) * g.dh + 1 + 0, PW = (g.OW - 1) * g.sw + (g.S - 1) * g.dw + 1;
    const bool staged_ok = (size_t)PH * PW * 4 <= 40 * 1024 && ((g.R == 5 && g.S == 5) || (g.R == 3 && g.S == 3)) &&
                           g.OH * g.OW >= 64;
    if (mtl_conv_wgrad_rows_supported(g, ug)) return mtl_conv_wgrad_bias_rows(ctx, dW, nullptr, ug, X, g, accumulate, 0);
    if (staged_ok) {
        constexpr int KB = 4;
        const int kgroups = (g.K + KB - 1) / KB;
        int ns = pick_nsplit(ctx, kgroups * g.C, g.N);
        int nps = (g.N + ns - 1) / ns;
        ns = (g.N + nps - 1) / nps;
        void* ws2;
        int32_t rc2 = mtl_workspace(ctx, (size_t)ns * kc * taps * 4, &ws2);
        if (rc2) return rc2;
        float* part = (float*)ws2;
        dim3 sgrid((unsigned)(kgroups * g.C), (unsigned)ns);
        size_t smem = (size_t)PH * PW * 4;
        if (g.R == 5) k_conv_wgrad_staged<5, 5, KB><<<sgrid, kBlock, smem, ctx->stream>>>(part, ug, X, g, nps, PH, PW);
        else k_conv_wgrad_staged<3, 3, KB><<<sgrid, kBlock, smem, ctx->stream>>>(part, ug, X, g, nps, PH, PW);
        MTL_LAUNCHED(ctx);
        return mtl_sum_partials(ctx, dW, part, (int64_t)kc * taps, ns, accumulate);
    }
    dim3 grid((unsigned)kc, (unsigned)nsplit);
    if (g.R == 5 && g.S == 5) k_conv_wgrad_taps<5, 5><<<grid, kBlock, 0, ctx->stream>>>(partial, ug, X, g, n_per_split);
    else if (g.R == 3 && g.S == 3) k_conv_wgrad_taps<3, 3><<<grid, kBlock, 0, ctx->stream>>>(partial, ug, X, g, n_per_split);
    else if (g.R == 1 && g.S == 1) k_conv_wgrad_taps<1, 1><<<grid, kBlock, 0, ctx->stream>>>(partial, ug, X, g, n_per_split);
    else k_conv_wgrad_generic<<<grid, kBlock, 0, ctx->stream>>>(partial, ug, X, g, n_per_split);
    MTL_LAUNCHED(ctx);
    return mtl_sum_partials(ctx, dW, partial, (int64_t)kc * taps, nsplit, accumulate);
}

int32_t mtl_conv_bgrad(mtl_ctx* ctx, float* db, const float* ug, const ConvGeom& g, int accumulate) {
    int nsplit = pick_nsplit(ctx, g.K, g.N);
    int n_per_split = (g.N + nsplit - 1) / nsplit;
    nsplit = (g.N + n_per_split - 1) / n_per_split;
    void* ws;
    int32_t rc = mtl_workspace(ctx, (size_t)nsplit * g.K * 4, &ws);
    if (rc) return rc;
    float* partial = (float*)ws;
    dim3 grid((unsigned)g.K, (unsigned)nsplit);
    k_conv_bgrad<<<grid, kBlock, 0, ctx->stream>>>(partial, ug, g.N, g.K, g.OH * g.OW, n_per_split);
    MTL_LAUNCHED(ctx);
    return mtl_sum_partials(ctx, db, partial, g.K, nsplit, accumulate);
}
