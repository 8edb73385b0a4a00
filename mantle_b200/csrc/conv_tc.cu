// OP.CONV2D on the tensor cores as implicit GEMM (stride 1, dilation 1):
//   forward      Y[(n,oh,ow), k]   = sum over (r,s,c) of X[n, oh+r-ph, ow+s-pw, c] * W[k, c, r, s]
//   input grad   dX[(n,ih,iw), c]  = the same form on ug with spatially flipped, transposed weights
// The activation tensor is first re-laid out channels-last (one pass, fused with the tf32 hi/lo
// split), so that one TMA box {32 channels, bw, bh, bn pixels} is a K-major 128-byte-swizzled
// operand tile; shifting the box origin by (r, s) walks the filter taps and the TMA zero fill
// outside the tensor is the convolution's zero padding.  Weights are re-laid out as [tap][out][in].
// Pipeline and warp roles are those of the DOT kernel: TMA producer warp, MMA issuer warp, four
// epilogue warps, two accumulators in tensor memory; the epilogue adds the bias and writes NCHW.
#include "conv.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128;
constexpr int BK = 32;
constexpr int kThreads = 192;
constexpr uint64_t kWaitBudgetNs = 4000000000ull;

template <int BN>
struct Cfg {
    static constexpr int kStages = BN == 128 ? 6 : 8;
    static constexpr int kABytes = BM * BK * 4;
    static constexpr int kBBytes = BN * BK * 4;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

struct ConvTcParams {
    int N, OH, OW, Kout;  // output [N, Kout, OH, OW]
    int Cin;              // channels reduced per tap
    int R, S, ph, pw;     // input pixel = output pixel + (r - ph, s - pw)
    int bw, bh, bn;       // pixel box of one tile, bw*bh*bn <= 128
    int tiles_w, tiles_h, tiles_nb, tiles_k;
    int nseg, segA[3], segB[3];
    uint32_t a_bytes;     // bytes one activation box delivers
    float* out;
    const float* bias;
    int accumulate;
    int32_t* status;
};

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
k_conv_igemm(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
             const __grid_constant__ CUtensorMap mapB0, const __grid_constant__ CUtensorMap mapB1, ConvTcParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + C::kStages;
    uint64_t* tmem_full = bars + 2 * C::kStages;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int tiles_m = p.tiles_w * p.tiles_h * p.tiles_nb;
    const int num_tiles = tiles_m * p.tiles_k;
    const int cblocks = (p.Cin + BK - 1) / BK;
    const int kb_per_seg = p.R * p.S * cblocks;
    const int kb_total = kb_per_seg * p.nseg;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&tmem_full[a], 1);
            mbar_init(&tmem_empty[a], 128);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&mapA0);
        prefetch_tensormap(&mapB0);
        if (p.nseg > 1) {
            prefetch_tensormap(&mapA1);
            prefetch_tensormap(&mapB1);
        }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    mtl_pdl_sync();   // everything above touched only shared / tensor memory

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int kt = t % p.tiles_k;
                int mt = t / p.tiles_k;
                const int tw = mt % p.tiles_w;
                mt /= p.tiles_w;
                const int th = mt % p.tiles_h;
                const int tnb = mt / p.tiles_h;
                const int ow0 = tw * p.bw, oh0 = th * p.bh, n0 = tnb * p.bn;
                for (int kb = 0; kb < kb_total; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, kWaitBudgetNs)) { ok = false; break; }
                    const int seg = kb / kb_per_seg;
                    int rem = kb - seg * kb_per_seg;
                    const int rs = rem / cblocks;
                    const int cb = rem - rs * cblocks;
                    const int r = rs / p.S, s = rs - r * p.S;
                    const CUtensorMap* ma = p.segA[seg] ? &mapA1 : &mapA0;
                    const CUtensorMap* mb = p.segB[seg] ? &mapB1 : &mapB0;
                    uint8_t* sa = tiles + stage * C::kStageBytes;
                    uint8_t* sb = sa + C::kABytes;
                    mbar_arrive_expect_tx(&full[stage], p.a_bytes + C::kBBytes);
                    tma_load_4d(sa, ma, &full[stage], cb * BK, ow0 + s - p.pw, oh0 + r - p.ph, n0);
                    tma_load_3d(sb, mb, &full[stage], cb * BK, kt * BN, rs);
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_tf32(BN, false, false);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int local = 0;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
                const int acc = local & 1;
                const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
                if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, kWaitBudgetNs)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < kb_total; ++kb) {
                    if (!mbar_wait(&full[stage], phase, abort_flag, kWaitBudgetNs)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(tiles + stage * C::kStageBytes);
                    const uint32_t sb = sa + C::kABytes;
#pragma unroll
                    for (int kk = 0; kk < BK / 8; ++kk) {
                        const uint64_t da = desc_k_major(sa, kk);
                        const uint64_t db = desc_k_major(sb, kk);
                        mma_tf32(tmem_d, da, db, idesc, (kb | kk) ? 1u : 0u);
                    }
                    mma_commit(&empty[stage]);
                    if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) mma_commit(&tmem_full[acc]);
            }
            if (!ok) atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else {
        const int quad = warp & 3;
        const int row = quad * 32 + lane;  // pixel slot inside the tile's box
        const int w_i = row % p.bw;
        const int h_i = (row / p.bw) % p.bh;
        const int n_i = row / (p.bw * p.bh);
        const int plane = p.OH * p.OW;
        bool ok = true;
        int local = 0;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
            const int kt = t % p.tiles_k;
            int mt = t / p.tiles_k;
            const int tw = mt % p.tiles_w;
            mt /= p.tiles_w;
            const int th = mt % p.tiles_h;
            const int tnb = mt / p.tiles_h;
            const int ow = tw * p.bw + w_i, oh = th * p.bh + h_i, n = tnb * p.bn + n_i;
            const bool valid = n_i < p.bn && ow < p.OW && oh < p.OH && n < p.N;
            const int acc = local & 1;
            const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
            if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, kWaitBudgetNs)) { ok = false; break; }
            tc_fence_after_sync();
            float* obase = p.out + ((int64_t)n * p.Kout) * plane + (int64_t)oh * p.OW + ow;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * BN + c * 32), r);
                tmem_ld_wait();
                const int k0 = kt * BN + c * 32;
                if (valid) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int k = k0 + j;
                        if (k < p.Kout) {
                            float v = __uint_as_float(r[j]);
                            if (p.bias) v += __ldg(p.bias + k);
                            float* dst = obase + (int64_t)k * plane;
                            *dst = p.accumulate ? *dst + v : v;
                        }
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&tmem_empty[acc]);
        }
        if (!ok && lane == 0) atomicExch(p.status, MTL_ERR_TIMEOUT);
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

__device__ __forceinline__ void split_tf32(float v, float& h, float& l) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
    h = __uint_as_float(u);
    l = v - h;
}

// [N, C, HW] -> [N, HW, C] through a 32x32 shared-memory tile; optionally also writes the residual.
// With `colsum` the block also leaves the sum of its 32 pixels for each of its 32 channels in
// colsum[(n * pixel_tiles + pixel_tile) * C + c]: the bias gradient read off the same pass.
template <bool SPLIT>
__global__ void __launch_bounds__(256) k_nchw_to_nhwc(float* __restrict__ hi, float* __restrict__ lo,
                                                      const float* __restrict__ X, int C, int HW,
                                                      float* __restrict__ colsum) {
    mtl_pdl_sync();
    __shared__ float tile[32][33];
    __shared__ float part[8][33];
    const int n = blockIdx.z;
    const int p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    const float* xin = X + (int64_t)n * C * HW;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int c = c0 + ty + 8 * i, pp = p0 + tx;
        tile[ty + 8 * i][tx] = (c < C && pp < HW) ? xin[(int64_t)c * HW + pp] : 0.0f;
    }
    __syncthreads();
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int pp = p0 + ty + 8 * i, c = c0 + tx;
        if (pp < HW && c < C) {
            float v = tile[tx][ty + 8 * i];
            s += v;
            int64_t o = ((int64_t)n * HW + pp) * C + c;
            if (SPLIT) {
                float h, l;
                split_tf32(v, h, l);
                hi[o] = h;
                lo[o] = l;
            } else {
                hi[o] = v;
            }
        }
    }
    if (colsum) {
        part[ty][tx] = s;
        __syncthreads();
        if (ty == 0 && c0 + tx < C) {
            float t = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) t += part[j][tx];
            colsum[((int64_t)n * gridDim.x + blockIdx.x) * C + c0 + tx] = t;
        }
    }
}

// out[y][c] (+)= sum over the rows of slice y of m[row][c]: 32 columns x 8 row lanes per block,
// coalesced row segments, fixed order of additions.  grid = (cols / 32, slices).
__global__ void __launch_bounds__(256) k_colsum(float* __restrict__ out, const float* __restrict__ m, int64_t rows,
                                                int cols, int64_t rows_per_slice, int accumulate) {
    mtl_pdl_sync();
    __shared__ float part[8][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + tx;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_slice;
    const int64_t r1 = r0 + rows_per_slice < rows ? r0 + rows_per_slice : rows;
    float s = 0.0f;
    if (c < cols) {
        int64_t r = r0 + ty;
        for (; r + 24 < r1; r += 32) {   // four rows in flight, added in the order a plain loop adds them
            const float a0 = m[r * cols + c], a1 = m[(r + 8) * cols + c], a2 = m[(r + 16) * cols + c], a3 = m[(r + 24) * cols + c];
            s += a0; s += a1; s += a2; s += a3;
        }
        for (; r < r1; r += 8) s += m[r * cols + c];
    }
    part[ty][tx] = s;
    __syncthreads();
    if (ty == 0 && c < cols) {
        float t = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) t += part[j][tx];
        float* o = out + (int64_t)blockIdx.y * cols + c;
        *o = accumulate ? *o + t : t;
    }
}

// MAXPOOL2D.backward (2x2 windows, stride 2) followed by RELU.backward, written CHANNELS-LAST: from the
// pooled upper gradient pg, the argmax indices and the pooled values pv (all [N, K, POH, POW]) to the
// dense gradient [N, 2*POH, 2*POW, K] the implicit-GEMM kernels read, split into hi / lo on the way
// when asked.  One block = one image x 32 channels: the pooled planes are read along their pixels
// (coalesced), kept in shared memory, and written along the channels (coalesced).  colsum as in
// k_nchw_to_nhwc: per-block channel sums, here colsum[n * K + k].
template <bool SPLIT>
__global__ void __launch_bounds__(256) k_pool_bwd_2x2_cl(float* __restrict__ hi, float* __restrict__ lo,
                                                         float* __restrict__ colsum, const float* __restrict__ pg,
                                                         const int32_t* __restrict__ pidx,
                                                         const float* __restrict__ pv, int K, int POH, int POW,
                                                         int relu) {
    mtl_pdl_sync();
    extern __shared__ float pool_smem[];
    const int P = POH * POW, PS = P | 1;   // odd row stride: lanes (channels) hit different banks
    float* val = pool_smem;                // [32][PS] gradient routed to the selected element
    int* pos = reinterpret_cast<int*>(pool_smem + 32 * PS);  // [32][PS] which of the four (0..3), -1 none
    __shared__ float part[8][33];
    const int n = blockIdx.y, c0 = blockIdx.x * 32;
    const int W = 2 * POW;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // Phase 1, a warp per channel row, lanes along the pooled plane (coalesced): which of its window's
    // four positions an element's gradient goes to, and the gradient after RELU.backward.  All offsets
    // inside one image fit 32 bits; the image's base pointers carry the 64-bit part.
    const float* pg_n = pg + (int64_t)n * K * P;
    const int32_t* pidx_n = pidx + (int64_t)n * K * P;
    const float* pv_n = relu ? pv + (int64_t)n * K * P : nullptr;
    for (int q0 = 0; q0 < P; q0 += 32) {
        const int q = q0 + lane;
        const int qh = q / POW, qw = q - qh * POW;
        const int first = (2 * qh) * W + 2 * qw;       // plane index of the window's upper left element
        if (q < P) {
#pragma unroll 4
            for (int ch = warp; ch < 32; ch += 8) {
                float v = 0.0f;
                int sub = -1;
                if (c0 + ch < K) {
                    const int o = (c0 + ch) * P + q;
                    v = pg_n[o];
                    if (relu) v = (pv_n[o] > 0.0f ? 1.0f : 0.0f) * v;   // RELU.backward on the selected element
                    const int d = pidx_n[o] - first;
                    sub = d == 0 ? 0 : d == 1 ? 1 : d == W ? 2 : d == W + 1 ? 3 : -1;
                }
                val[ch * PS + q] = v;
                pos[ch * PS + q] = sub;
            }
        }
    }
    __syncthreads();
    // Phase 2, lanes along the channels (coalesced channels-last stores): a warp takes a window at a
    // time and writes its four pixels, the routed gradient in one of them and zeros in the others.
    const int k = c0 + lane;
    float s = 0.0f;
    float* hi_n = hi + (int64_t)n * 4 * P * K;
    float* lo_n = SPLIT ? lo + (int64_t)n * 4 * P * K : nullptr;
    const int row = W * K;                          // one output row of the image, channels-last
    int qh = warp / POW, qw = warp - qh * POW;      // window (qh, qw) = window number `warp`, then + 8 each turn
    for (int q = warp; q < P; q += 8) {
        const float g = val[lane * PS + q];
        const int sub = pos[lane * PS + q];
        s += sub >= 0 ? g : 0.0f;
        if (k < K) {
            const int o = (2 * qh) * row + 2 * qw * K + k;
            const float v0 = sub == 0 ? g : 0.0f, v1 = sub == 1 ? g : 0.0f, v2 = sub == 2 ? g : 0.0f, v3 = sub == 3 ? g : 0.0f;
            if (SPLIT) {
                float h, l;
                split_tf32(v0, h, l); hi_n[o] = h; lo_n[o] = l;
                split_tf32(v1, h, l); hi_n[o + K] = h; lo_n[o + K] = l;
                split_tf32(v2, h, l); hi_n[o + row] = h; lo_n[o + row] = l;
                split_tf32(v3, h, l); hi_n[o + row + K] = h; lo_n[o + row + K] = l;
            } else {
                hi_n[o] = v0;
                hi_n[o + K] = v1;
                hi_n[o + row] = v2;
                hi_n[o + row + K] = v3;
            }
        }
        qw += 8;
        while (qw >= POW) { qw -= POW; ++qh; }
    }
    if (colsum) {
        part[warp][lane] = s;
        __syncthreads();
        if (warp == 0 && k < K) {
            float t = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) t += part[j][lane];
            colsum[(int64_t)n * K + k] = t;
        }
    }
}

// Weights [K, C, R, S] -> forward layout [tap][K][C], or (flip) input-gradient layout
// [flipped tap][C][K].
template <bool SPLIT>
__global__ void __launch_bounds__(256) k_weights_relayout(float* __restrict__ hi, float* __restrict__ lo,
                                                          const float* __restrict__ Wt, int K, int C, int R, int S,
                                                          int flip) {
    mtl_pdl_sync();
    int64_t total = (int64_t)K * C * R * S;
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t o = tid; o < total; o += stride) {
        int inner = flip ? K : C, mid = flip ? C : K;
        int i0 = (int)(o % inner);
        int64_t q = o / inner;
        int i1 = (int)(q % mid);
        int rs = (int)(q / mid);
        int r = rs / S, s = rs - r * S;
        int k = flip ? i0 : i1, c = flip ? i1 : i0;
        if (flip) { r = R - 1 - r; s = S - 1 - s; }
        float v = Wt[(((int64_t)k * C + c) * R + r) * S + s];
        if (SPLIT) {
            float h, l;
            split_tf32(v, h, l);
            hi[o] = h;
            lo[o] = l;
        } else {
            hi[o] = v;
        }
    }
}

// Paired layout for layers with at most 64 output channels: [r * SP + sp][128 rows][inner], row
// 32 * q + 16 * h + j holding channel 16 * q + j of logical tap (r, 2 * sp + h); rows past the channel
// count and the missing partner of an odd last tap are zero.  SP = ceil(S / 2).
// pair == 0 ("spread"): one tap per slot, half 1 all zero -- only the row order is used, so that the
// (at most 64) channels are shared by all four epilogue warps.
template <bool SPLIT>
__global__ void __launch_bounds__(256) k_weights_relayout_paired(float* __restrict__ hi, float* __restrict__ lo,
                                                                 const float* __restrict__ Wt, int K, int C, int R,
                                                                 int S, int flip, int pair) {
    mtl_pdl_sync();
    const int SP = pair ? (S + 1) / 2 : S;
    const int inner = flip ? K : C, mid = flip ? C : K;
    int64_t total = (int64_t)R * SP * 128 * inner;
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t o = tid; o < total; o += stride) {
        int i0 = (int)(o % inner);
        int64_t q = o / inner;
        int row = (int)(q % 128);
        int g = (int)(q / 128);
        // rows are grouped per 32 (one TMEM lane quadrant = one epilogue warp): 16 channels of half 0,
        // then the same 16 channels of half 1, so that the two halves of a channel meet in one warp
        int h = (row >> 4) & 1, i1 = (row >> 5) * 16 + (row & 15);
        int r = g / SP, s = pair ? 2 * (g - r * SP) + h : g - r * SP;
        float v = 0.0f;
        if (i1 < mid && s < S && (pair || h == 0)) {
            int k = flip ? i0 : i1, c = flip ? i1 : i0;
            int rr = flip ? R - 1 - r : r, ss = flip ? S - 1 - s : s;
            v = Wt[(((int64_t)k * C + c) * R + rr) * S + ss];
        }
        if (SPLIT) {
            float hh, ll;
            split_tf32(v, hh, ll);
            hi[o] = hh;
            lo[o] = ll;
        } else {
            hi[o] = v;
        }
    }
}

// Picks the pixel box {bw, bh, bn} (product <= 128) that wastes the fewest accumulator rows.
void choose_box(int OW, int OH, int N, int* bw_, int* bh_, int* bn_) {
    double best = -1.0;
    int bbw = 1, bbh = 1, bbn = 1;
    for (int bw = 1; bw <= OW && bw <= 128; ++bw) {
        for (int bh = 1; bh <= OH && bw * bh <= 128; ++bh) {
            int bn = 128 / (bw * bh);
            if (bn > N) bn = N;
            if (bn > 128) bn = 128;
            int64_t tiles = (int64_t)((OW + bw - 1) / bw) * ((OH + bh - 1) / bh) * ((N + bn - 1) / bn);
            double eff = (double)OW * OH * N / ((double)tiles * 128.0);
            // prefer long contiguous output runs at equal efficiency
            double score = eff + 1e-4 * bw;
            if (score > best) { best = score; bbw = bw; bbh = bh; bbn = bn; }
        }
    }
    *bw_ = bbw; *bh_ = bbh; *bn_ = bbn;
}

struct IgemmCall {
    // logical problem: out[N, Kout, OH, OW] from act[N, Cin, IH, IW] (NCHW in memory)
    int N, Cin, IH, IW, Kout, OH, OW, R, S, ph, pw;
    const float* act;   // NCHW activations (X or ug)
    const float* wt;    // [K, C, R, S] weights as the reference stores them
    int wK, wC;         // the K and C extents of `wt`
    int flip;           // 0 forward, 1 input gradient
    float* out;
    const float* bias;
    int accumulate;
    int relu;           // clamp the result at zero after the bias (forward with a fused RELU)
    const float* act_cl = nullptr;  // channels-last copy of `act` the caller already has (plain TF32 only)
    int pool = 0;                   // 2x2 / stride-2 max pooling in the epilogue: out = pooled values
    int32_t* pool_idx = nullptr;    // argmax indices of that pooling (may be null)
};

// ------------------------------------------------------------------ channel-major variant -----
// Measured on B200: one tcgen05.mma kind::tf32 with M = 128 costs about 71 ns + 0.164 ns * N, i.e.
// fetching the A operand is a large fixed cost and the instruction only reaches the tensor peak
// near N = 256.  Output channels (64..128 per layer here) therefore go on the M axis and the
// PIXELS on the N axis: A = one weight tile {128 out-ch x 32 in-ch}, B = up to 256 pixels x 32
// in-ch fetched by one TMA box {32, bw, bh, bn}.  Accumulator D[out-ch, pixel]: a thread of the
// epilogue owns one output channel and walks the tile's pixels, which are contiguous in NCHW.
constexpr int kTStages = 4;
constexpr int kTABytes = BM * BK * 4;        // weights tile
constexpr int kTBBytes = 256 * BK * 4;       // pixel tile (maximum)
constexpr int kTStageBytes = kTABytes + kTBBytes;
constexpr int kTStgFloats = 32 * 36;  // per epilogue warp: transposition block
constexpr int kTSmemBytes = kTStages * kTStageBytes + 1024 + 256 + 256 * 4 + 64 * 4 + 4 * kTStgFloats * 4;

struct ConvTParams {
    int N, OH, OW, Kout, Cin;
    int R, S, ph, pw;
    int bw, bh, bn, npix;   // pixel box, npix = bw*bh*bn <= 256
    int n_mma;              // npix rounded up to a multiple of 16: the N extent of the instruction
    int tiles_w, tiles_h, tiles_nb, tiles_k;
    int nseg, segA[3], segB[3];
    float* out;
    const float* bias;
    int accumulate;
    int relu;
    // 2x2 / stride-2 max pooling in the epilogue (box = whole rows, two of them, at most 32 pixels per
    // image): `out` then receives the pooled values [N, Kout, OH/2, OW/2] and pool_idx the argmax indices
    // (plane-local, MAXPOOL2D.forward's strict '>' scan in row-major window order, pool.mojo:44-100)
    int pool;
    int32_t* pool_idx;
    // Tap pairing (at most 64 output channels): of every 32 rows of the weight tile, 16 hold tap
    // (r, 2*si) of 16 channels and 16 hold tap (r, 2*si + 1) of the same channels; both see the pixel
    // box of the first tap, so the second half of the accumulator is the second tap's contribution to
    // the pixel one column to the LEFT, and the epilogue adds half1[column + 1] to half0[column] with
    // a warp shuffle.  The box is one column wider than the image.
    int paired;             // 0 off, 1 two taps per instruction, 2 only the row order ("spread": no second tap)
    int s_count, s_step;    // iterations over the kernel width and their tap stride (1, or 2 when paired)
    int acc_stride;         // TMEM columns between the two accumulators (248 when paired: the shifted
                            // read of the second one must stay inside the 512 allocated columns)
    int vec_ok;             // channel planes are 16-byte aligned: four adjacent pixels may leave as a float4
    // Work items: the first `whole_items` are whole tiles; every later pair is ONE tile whose k-blocks are
    // split at kb_half over two CTAs (the tiles of a partial last wave, when twice as many CTAs are free).
    // Each half parks its accumulator in split_scratch unless the other half is already there; whichever
    // finishes second adds the parked half to its own (a + b == b + a, so the result does not depend on
    // which one that was) and runs the ordinary epilogue.
    int whole_items, n_items, kb_half;
    float4* split_scratch;      // per split tile and half: [16 column chunks][4 warps][4][32 lanes] float4
    int32_t* split_tickets;     // per split tile, zero between launches
    int32_t* status;
};

struct ConvTItem {
    int tile, kb0, kb1, slot, part;   // slot < 0: a whole tile
};
__device__ __forceinline__ ConvTItem conv_t_item(const ConvTParams& p, int w, int kb_total) {
    ConvTItem it;
    if (w < p.whole_items) {
        it.tile = w; it.kb0 = 0; it.kb1 = kb_total; it.slot = -1; it.part = 0;
    } else {
        const int i = w - p.whole_items;
        it.slot = i >> 1; it.part = i & 1; it.tile = p.whole_items + it.slot;
        it.kb0 = it.part ? p.kb_half : 0;
        it.kb1 = it.part ? kb_total : p.kb_half;
    }
    return it;
}

// 2x2 / stride-2 max pooling of one channel's BW x 2 pixels held in registers (r[0..BW) the upper row,
// r[BW..2BW) the lower), after bias and RELU.  MAXPOOL2D.forward order: the window is scanned
// row-major with a strict '>', so the first of equal values wins.  Values and argmax indices go to
// shared memory at [channel * 9 + column] (stride 9 keeps both the writes and the reads spread
// over the banks).
template <int BW>
__device__ __forceinline__ void pool_rows_in_registers(const uint32_t (&r)[32], float bv, int relu, int i00, int OW,
                                                       float* pv, int32_t* pi) {
#pragma unroll
    for (int pw = 0; pw < BW / 2; ++pw) {
        float a = __uint_as_float(r[2 * pw]) + bv, b = __uint_as_float(r[2 * pw + 1]) + bv;
        float c = __uint_as_float(r[BW + 2 * pw]) + bv, d = __uint_as_float(r[BW + 2 * pw + 1]) + bv;
        if (relu) {
            a = a > 0.0f ? a : 0.0f; b = b > 0.0f ? b : 0.0f;
            c = c > 0.0f ? c : 0.0f; d = d > 0.0f ? d : 0.0f;
        }
        float m = -INFINITY;
        int j = -1;
        const int i = i00 + 2 * pw;
        if (a > m) { m = a; j = i; }
        if (b > m) { m = b; j = i + 1; }
        if (c > m) { m = c; j = i + OW; }
        if (d > m) { m = d; j = i + OW + 1; }
        pv[pw] = m;
        pi[pw] = j;
    }
}

__global__ void __launch_bounds__(kThreads, 1)
k_conv_igemm_t(const __grid_constant__ CUtensorMap mapX0, const __grid_constant__ CUtensorMap mapX1,
               const __grid_constant__ CUtensorMap mapW0, const __grid_constant__ CUtensorMap mapW1, ConvTParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kTStages * kTStageBytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + kTStages;
    uint64_t* tmem_full = bars + 2 * kTStages;
    uint64_t* tmem_empty = tmem_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* split_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
    int* col_off = reinterpret_cast<int*>(smem + kTStages * kTStageBytes + 256);
    int* col_vec = col_off + 256;
    float* stage_buf = reinterpret_cast<float*>(col_vec + 64);  // 4 warps x kTStgFloats

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cblocks = (p.Cin + BK - 1) / BK;
    const int kb_per_seg = p.R * p.s_count * cblocks;
    const int kb_total = kb_per_seg * p.nseg;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 128); }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&mapX0);
        prefetch_tensormap(&mapW0);
        if (p.nseg > 1) { prefetch_tensormap(&mapX1); prefetch_tensormap(&mapW1); }
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    mtl_pdl_sync();   // everything above touched only shared / tensor memory

    if (warp == 0) {
        // two producer lanes: issuing a TMA copy occupies its thread for a few hundred cycles, so the
        // weight box (lane 0) and the pixel box (lane 1) of a stage are issued side by side
        if (lane < 2) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const uint32_t tx = (uint32_t)kTABytes + (uint32_t)p.npix * 128u;
            for (int w = blockIdx.x; w < p.n_items && ok; w += gridDim.x) {
                const ConvTItem it = conv_t_item(p, w, kb_total);
                const int t = it.tile;
                const int kt = t % p.tiles_k;
                int mt = t / p.tiles_k;
                const int tw = mt % p.tiles_w;
                mt /= p.tiles_w;
                const int th = mt % p.tiles_h;
                const int tnb = mt / p.tiles_h;
                const int ow0 = tw * p.bw, oh0 = th * p.bh, n0 = tnb * p.bn;
                if (it.slot < 0) {
                    // a whole tile: plain nested loops (measured: walking them through one flat k-block counter,
                    // as the split items below do, made this kernel 6 - 12 % slower -- the producer's issue rate
                    // is on the critical path)
                    for (int seg = 0; seg < p.nseg && ok; ++seg) {
                        const CUtensorMap* mx = p.segA[seg] ? &mapX1 : &mapX0;
                        const CUtensorMap* mw = p.segB[seg] ? &mapW1 : &mapW0;
                        for (int r = 0; r < p.R && ok; ++r)
                            for (int si = 0; si < p.s_count && ok; ++si)
                                for (int cb = 0; cb < cblocks; ++cb) {
                                    if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, kWaitBudgetNs)) ok = false;
                                    if (__any_sync(0x3u, !ok)) { ok = false; break; }
                                    uint8_t* sa = tiles + stage * kTStageBytes;
                                    uint8_t* sb = sa + kTABytes;
                                    if (lane == 0) mbar_arrive_expect_tx(&full[stage], tx);
                                    __syncwarp(0x3u);
                                    if (lane == 0) tma_load_3d(sa, mw, &full[stage], cb * BK, kt * BM, r * p.s_count + si);
                                    else tma_load_4d(sb, mx, &full[stage], cb * BK, ow0 + si * p.s_step - p.pw, oh0 + r - p.ph, n0);
                                    if (++stage == kTStages) { stage = 0; phase ^= 1u; }
                                }
                    }
                    continue;
                }
                // k-block kb = ((seg * R + r) * s_count + si) * cblocks + cb
                int seg = it.kb0 / kb_per_seg;
                int rest = it.kb0 - seg * kb_per_seg;
                int r = rest / (p.s_count * cblocks);
                rest -= r * p.s_count * cblocks;
                int si = rest / cblocks;
                int cb = rest - si * cblocks;
                for (int kb = it.kb0; kb < it.kb1; ++kb) {
                    const CUtensorMap* mx = p.segA[seg] ? &mapX1 : &mapX0;
                    const CUtensorMap* mw = p.segB[seg] ? &mapW1 : &mapW0;
                    if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, kWaitBudgetNs)) ok = false;
                    if (__any_sync(0x3u, !ok)) { ok = false; break; }
                    uint8_t* sa = tiles + stage * kTStageBytes;
                    uint8_t* sb = sa + kTABytes;
                    if (lane == 0) mbar_arrive_expect_tx(&full[stage], tx);
                    __syncwarp(0x3u);
                    if (lane == 0) tma_load_3d(sa, mw, &full[stage], cb * BK, kt * BM, r * p.s_count + si);
                    else tma_load_4d(sb, mx, &full[stage], cb * BK, ow0 + si * p.s_step - p.pw, oh0 + r - p.ph, n0);
                    if (++stage == kTStages) { stage = 0; phase ^= 1u; }
                    if (++cb == cblocks) {
                        cb = 0;
                        if (++si == p.s_count) {
                            si = 0;
                            if (++r == p.R) { r = 0; ++seg; }
                        }
                    }
                }
            }
            if (!ok && lane == 0) atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = make_idesc_tf32(p.n_mma, false, false);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int local = 0;
            for (int w = blockIdx.x; w < p.n_items && ok; w += gridDim.x, ++local) {
                const ConvTItem it = conv_t_item(p, w, kb_total);
                const int acc = local & 1;
                const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
                if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, kWaitBudgetNs)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * p.acc_stride);
                for (int kb = it.kb0; kb < it.kb1; ++kb) {
                    if (!mbar_wait(&full[stage], phase, abort_flag, kWaitBudgetNs)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(tiles + stage * kTStageBytes);
                    const uint32_t sb = sa + kTABytes;
#pragma unroll
                    for (int kk = 0; kk < BK / 8; ++kk)
                        mma_tf32(tmem_d, desc_k_major(sa, kk), desc_k_major(sb, kk), idesc, (kb > it.kb0 || kk) ? 1u : 0u);
                    mma_commit(&empty[stage]);
                    if (++stage == kTStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) mma_commit(&tmem_full[acc]);
            }
            if (!ok) atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else {
        const int quad = warp & 3;
        const int krow = quad * 32 + lane;  // output channel inside the tile
        const int plane = p.OH * p.OW;
        bool ok = true;
        int local = 0;
        for (int w = blockIdx.x; w < p.n_items && ok; w += gridDim.x, ++local) {
            const ConvTItem it = conv_t_item(p, w, kb_total);
            const int t = it.tile;
            const int kt = t % p.tiles_k;
            int mt = t / p.tiles_k;
            const int tw = mt % p.tiles_w;
            mt /= p.tiles_w;
            const int th = mt % p.tiles_h;
            const int tnb = mt / p.tiles_h;
            const int ow0 = tw * p.bw, oh0 = th * p.bh, n0 = tnb * p.bn;
            // paired: this warp's 32 rows are 16 channels twice (see k_weights_relayout_paired)
            const int k = p.paired ? quad * 16 + (lane & 15) : kt * BM + krow;
            const bool kvalid = k < p.Kout && (!p.paired || lane < 16);
            const float bv = (kvalid && p.bias) ? __ldg(p.bias + k) : 0.0f;
            const int acc = local & 1;
            const uint32_t acc_phase = (uint32_t)(local >> 1) & 1u;
            if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, kWaitBudgetNs)) { ok = false; break; }
            tc_fence_after_sync();
            if (it.slot >= 0) {
                // One half of a k-split tile.  Nobody waits here: a half that finds the other already parked
                // skips its own dump, otherwise it parks its accumulator and draws a ticket; the second to
                // draw adds the parked half into its own tensor memory and carries on as if it had run the
                // whole reduction.
                const uint32_t half_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * p.acc_stride);
                const int nchunk = p.n_mma >> 4;
                float4* mine = p.split_scratch + (size_t)(it.slot * 2 + it.part) * (16 * 4 * 4 * 32);
                const float4* other = p.split_scratch + (size_t)(it.slot * 2 + (it.part ^ 1)) * (16 * 4 * 4 * 32);
                int32_t* ticket = p.split_tickets + it.slot;
                if (threadIdx.x == 64) *split_flag = *reinterpret_cast<volatile int32_t*>(ticket);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                int folder = *split_flag;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!folder) {
                    // the read of the next 16 columns is issued before the current ones are stored
                    uint32_t v[2][16];
                    tmem_ld_32x16(half_addr, v[0]);
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        if (c < nchunk) {
                            tmem_ld_wait();
                            if (c + 1 < nchunk) tmem_ld_32x16(half_addr + (uint32_t)((c + 1) * 16), v[(c + 1) & 1]);
                            float4* dst = mine + ((size_t)(c * 4 + quad) * 4) * 32 + lane;
#pragma unroll
                            for (int g = 0; g < 4; ++g)
                                __stcg(dst + g * 32, make_float4(__uint_as_float(v[c & 1][g * 4]), __uint_as_float(v[c & 1][g * 4 + 1]),
                                                                 __uint_as_float(v[c & 1][g * 4 + 2]), __uint_as_float(v[c & 1][g * 4 + 3])));
                        }
                    }
                    __threadfence();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (threadIdx.x == 64) *split_flag = atomicAdd(ticket, 1);
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    folder = *split_flag;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                }
                if (!folder) {
                    tc_fence_before_sync();
                    mbar_arrive(&tmem_empty[acc]);
                    continue;
                }
                __threadfence();
                {
                    // The parked half comes from L2 (most of a microsecond per round trip): the loads of four
                    // 16-column chunks are kept in flight, a chunk's registers being refilled as soon as it has
                    // been added into tensor memory.
                    float4 o[4][4];
                    auto fetch_chunk = [&](int c, float4 (&dst)[4]) {
                        const float4* src = other + ((size_t)(c * 4 + quad) * 4) * 32 + lane;
#pragma unroll
                        for (int g = 0; g < 4; ++g) dst[g] = __ldcg(src + g * 32);
                    };
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (c < nchunk) fetch_chunk(c, o[c]);
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        if (c < nchunk) {
                            uint32_t v[16];
                            tmem_ld_32x16(half_addr + (uint32_t)(c * 16), v);
                            tmem_ld_wait();
#pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                v[g * 4] = __float_as_uint(__uint_as_float(v[g * 4]) + o[c & 3][g].x);
                                v[g * 4 + 1] = __float_as_uint(__uint_as_float(v[g * 4 + 1]) + o[c & 3][g].y);
                                v[g * 4 + 2] = __float_as_uint(__uint_as_float(v[g * 4 + 2]) + o[c & 3][g].z);
                                v[g * 4 + 3] = __float_as_uint(__uint_as_float(v[g * 4 + 3]) + o[c & 3][g].w);
                            }
                            tmem_st_32x16(half_addr + (uint32_t)(c * 16), v);
                            if (c + 4 < nchunk) fetch_chunk(c + 4, o[c & 3]);
                        }
                    }
                }
                tmem_st_wait();
                if (threadIdx.x == 64) *ticket = 0;   // ready for the next launch
            }
            // Column j of the accumulator is pixel (j % bw, (j / bw) % bh, j / (bw*bh)) of the box.
            // The 128 epilogue threads first tabulate, per column, the offset of that pixel inside
            // one channel plane set (-1 = outside the tensor) and, per group of four columns,
            // whether the four are contiguous and 16-byte aligned; the store loop then costs a few
            // instructions per column, which matters because only four warps drain 256 columns.
            asm volatile("bar.sync 1, 128;" ::: "memory");
            for (int j = (int)threadIdx.x - 64; j < 256; j += 128) {
                int o = -1;
                if (j < p.npix) {
                    const int w_i = j % p.bw, h_i = (j / p.bw) % p.bh, n_i = j / (p.bw * p.bh);
                    const int ow = ow0 + w_i, oh = oh0 + h_i, n = n0 + n_i;
                    if (ow < p.OW && oh < p.OH && n < p.N) o = n * p.Kout * plane + oh * p.OW + ow;
                }
                col_off[j] = o;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if ((int)threadIdx.x - 64 < 64) {
                const int g = (int)threadIdx.x - 64;
                const int o0 = col_off[g * 4], o1 = col_off[g * 4 + 1], o2 = col_off[g * 4 + 2], o3 = col_off[g * 4 + 3];
                col_vec[g] = (o0 >= 0 && o1 == o0 + 1 && o2 == o0 + 2 && o3 == o0 + 3 && (o0 & 3) == 0 && p.vec_ok) ? 1 : 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            // A thread of the accumulator owns one channel, but channels are a whole plane apart in
            // NCHW: storing from that layout scatters every warp store over 32 lines (measured: the
            // stores then take as long as the whole main loop).  Each warp therefore turns its
            // 32 channels x 32 pixels block through shared memory so that eight lanes write 32
            // adjacent pixels of one channel.
            float* stg = stage_buf + (warp - 2) * kTStgFloats;
            const int sub = lane & 7, chl = lane >> 3;
            if (p.pool) {
                // One image of the box at a time: its bw x 2 pixels are adjacent accumulator columns.
                // Each thread parks its channel's pixels in shared memory; then eight lanes take the
                // (up to) eight pooled columns of one channel, so a warp store covers four channels'
                // pooled rows.  MAXPOOL2D.forward order: window scanned row-major, strict '>', first wins.
                const int P = p.bw * p.bh, PWD = p.bw >> 1, POH = p.OH >> 1;
                float* prow = stg + lane * 33;
                const int poh = oh0 >> 1;
                const int i00 = oh0 * p.OW + 2 * sub;
                const bool pw_ok = sub < PWD;
                const bool in_regs = p.bw == 14 || p.bw == 16 || p.bw == 12 || p.bw == 8;
#pragma unroll 1
                for (int n_i = 0; n_i < p.bn; ++n_i) {
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * p.acc_stride + n_i * P), r);
                    tmem_ld_wait();
                    __syncwarp();
                    const int n = n0 + n_i;
                    const int kk0 = kt * BM + quad * 32 + chl;
                    int64_t o = (((int64_t)n * p.Kout + kk0) * POH + poh) * PWD + sub;
                    const int64_t ostep = (int64_t)4 * POH * PWD;
                    if (in_regs) {
                        float* pv = stg + lane * 9;
                        int32_t* pi = reinterpret_cast<int32_t*>(stg + 32 * 9) + lane * 9;
                        const int ib = oh0 * p.OW;
                        if (p.bw == 14) pool_rows_in_registers<14>(r, bv, p.relu, ib, p.OW, pv, pi);
                        else if (p.bw == 16) pool_rows_in_registers<16>(r, bv, p.relu, ib, p.OW, pv, pi);
                        else if (p.bw == 12) pool_rows_in_registers<12>(r, bv, p.relu, ib, p.OW, pv, pi);
                        else pool_rows_in_registers<8>(r, bv, p.relu, ib, p.OW, pv, pi);
                        __syncwarp();
                        if (n < p.N && pw_ok) {
                            float m[8];
                            int at[8];
#pragma unroll
                            for (int it = 0; it < 8; ++it) {
                                m[it] = stg[(it * 4 + chl) * 9 + sub];
                                at[it] = reinterpret_cast<const int32_t*>(stg + 32 * 9)[(it * 4 + chl) * 9 + sub];
                            }
#pragma unroll
                            for (int it = 0; it < 8; ++it, o += ostep) {
                                if (kk0 + it * 4 < p.Kout) {
                                    p.out[o] = m[it];
                                    if (p.pool_idx) p.pool_idx[o] = at[it];
                                }
                            }
                        }
                        continue;
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float v = __uint_as_float(r[j]) + bv;
                        if (p.relu) v = v > 0.0f ? v : 0.0f;
                        prow[j] = v;
                    }
                    __syncwarp();
                    if (n < p.N && pw_ok) {
                        float m[8];
                        int at[8];
#pragma unroll
                        for (int it = 0; it < 8; ++it) {
                            const float* q = stg + (it * 4 + chl) * 33 + 2 * sub;
                            const float a = q[0], b = q[1], c = q[p.bw], d = q[p.bw + 1];
                            float mm = -INFINITY;
                            int j = -1;
                            if (a > mm) { mm = a; j = i00; }
                            if (b > mm) { mm = b; j = i00 + 1; }
                            if (c > mm) { mm = c; j = i00 + p.OW; }
                            if (d > mm) { mm = d; j = i00 + p.OW + 1; }
                            m[it] = mm; at[it] = j;
                        }
#pragma unroll
                        for (int it = 0; it < 8; ++it, o += ostep) {
                            if (kk0 + it * 4 < p.Kout) {
                                p.out[o] = m[it];
                                if (p.pool_idx) p.pool_idx[o] = at[it];
                            }
                        }
                    }
                }
                tc_fence_before_sync();
                mbar_arrive(&tmem_empty[acc]);
                continue;
            }
            // The accumulator leaves tensor memory 32 columns at a time.  The read of the NEXT 32 columns is
            // issued as soon as the current ones are parked in shared memory, so that its latency runs under
            // the transposed read-back and the global stores of the current block (with short reductions this
            // epilogue, not the main loop, sets the pace of the kernel).
            uint32_t r[32], r2[32];
            const uint32_t acc_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * p.acc_stride);
            tmem_ld_32x32(acc_addr, r);
            if (p.paired == 1) tmem_ld_32x32(acc_addr + 1u, r2);
#pragma unroll 1
            for (int c = 0; c * 32 < p.npix; ++c) {
                tmem_ld_wait();
                if (p.paired == 1) {
                    // lanes 16-31 hold the second tap of the channels of lanes 0-15, which belongs to the pixel
                    // one column to the left: those lanes take their values one column to the right (r2).  The
                    // two halves meet in the transposition block below (row ch and row ch + 16), where the
                    // reading side adds them -- no warp shuffles, which would compete with the main loop for
                    // the shared-memory pipe.
                    if (lane >= 16) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = r2[i];
                    }
                }
                __syncwarp();
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    float4 o = make_float4(__uint_as_float(r[g * 4]) + bv, __uint_as_float(r[g * 4 + 1]) + bv,
                                           __uint_as_float(r[g * 4 + 2]) + bv, __uint_as_float(r[g * 4 + 3]) + bv);
                    if (p.relu && p.paired != 1) {  // RELU.forward: x > 0 ? x : 0 (paired: after the halves are added)
                        o.x = o.x > 0.0f ? o.x : 0.0f; o.y = o.y > 0.0f ? o.y : 0.0f;
                        o.z = o.z > 0.0f ? o.z : 0.0f; o.w = o.w > 0.0f ? o.w : 0.0f;
                    }
                    *reinterpret_cast<float4*>(stg + lane * 36 + g * 4) = o;
                }
                if ((c + 1) * 32 < p.npix) {
                    tmem_ld_32x32(acc_addr + (uint32_t)((c + 1) * 32), r);
                    if (p.paired == 1) tmem_ld_32x32(acc_addr + (uint32_t)((c + 1) * 32 + 1), r2);
                }
                __syncwarp();
                const int j0 = c * 32 + sub * 4;
                const int vec = col_vec[j0 >> 2];
                const int o0 = col_off[j0], o1 = col_off[j0 + 1], o2 = col_off[j0 + 2], o3 = col_off[j0 + 3];
                {
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int ch = it * 4 + chl;
                        const int kk = p.paired ? quad * 16 + ch : kt * BM + quad * 32 + ch;
                        if (kk < p.Kout && (!p.paired || ch < 16)) {
                            float4 val = *reinterpret_cast<const float4*>(stg + ch * 36 + sub * 4);
                            if (p.paired == 1) {
                                const float4 v2 = *reinterpret_cast<const float4*>(stg + (ch + 16) * 36 + sub * 4);
                                val.x += v2.x; val.y += v2.y; val.z += v2.z; val.w += v2.w;
                                if (p.relu) {
                                    val.x = val.x > 0.0f ? val.x : 0.0f; val.y = val.y > 0.0f ? val.y : 0.0f;
                                    val.z = val.z > 0.0f ? val.z : 0.0f; val.w = val.w > 0.0f ? val.w : 0.0f;
                                }
                            }
                            float* base = p.out + (int64_t)kk * plane;
                            if (vec) {
                                float4* dst = reinterpret_cast<float4*>(base + o0);
                                float4 o = val;
                                if (p.accumulate) {
                                    float4 old = *dst;
                                    o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                                }
                                *dst = o;
                            } else {
                                if (o0 >= 0) base[o0] = p.accumulate ? base[o0] + val.x : val.x;
                                if (o1 >= 0) base[o1] = p.accumulate ? base[o1] + val.y : val.y;
                                if (o2 >= 0) base[o2] = p.accumulate ? base[o2] + val.z : val.z;
                                if (o3 >= 0) base[o3] = p.accumulate ? base[o3] + val.w : val.w;
                            }
                        }
                    }
                }
            }
            tc_fence_before_sync();
            mbar_arrive(&tmem_empty[acc]);
        }
        if (!ok && lane == 0) atomicExch(p.status, MTL_ERR_TIMEOUT);
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

// Pixel box {bw, bh, bn} with at most `limit` pixels.  Among the boxes within 8 % of the best
// column utilisation, take the one whose pixels form the longest contiguous run in an NCHW plane
// (whole rows, then adjacent rows), because the epilogue stores runs; then the fuller one.
void choose_box_n(int OW, int OH, int N, int limit, int* bw_, int* bh_, int* bn_) {
    double best_eff = 0.0;
    for (int pass = 0; pass < 2; ++pass) {
        double best_score = -1.0;
        for (int bw = 1; bw <= OW && bw <= limit; ++bw)
            for (int bh = 1; bh <= OH && bw * bh <= limit; ++bh) {
                int bn = limit / (bw * bh);
                if (bn > N) bn = N;
                if (bn > 256) bn = 256;
                int64_t tiles = (int64_t)((OW + bw - 1) / bw) * ((OH + bh - 1) / bh) * ((N + bn - 1) / bn);
                double eff = (double)OW * OH * N / ((double)tiles * limit);
                if (pass == 0) {
                    if (eff > best_eff) best_eff = eff;
                    continue;
                }
                if (eff < 0.92 * best_eff) continue;
                int run = (bw == OW) ? bw * bh : bw;
                double score = run + eff;
                if (score > best_score) { best_score = score; *bw_ = bw; *bh_ = bh; *bn_ = bn; }
            }
    }
}

// k_conv_igemm_t's work items: the tiles of a partial last wave are split along k over two CTAs each when
// twice as many CTAs are free and the reduction is long enough to be worth a trip of one accumulator
// through L2 (put at an eighth of a tile in the cost of a plan).
static bool igemm_tail_splits(const mtl_ctx* ctx, int64_t tiles, int kblocks) {
    const int64_t rem = tiles % ctx->sm_count;
    return ctx->tune.conv_tail_split && rem > 0 && 2 * rem <= ctx->sm_count && kblocks >= 16;
}
static double igemm_waves(const mtl_ctx* ctx, int64_t tiles, int kblocks) {
    const int64_t full = tiles / ctx->sm_count, rem = tiles % ctx->sm_count;
    if (rem == 0) return (double)full;
    return (double)full + (igemm_tail_splits(ctx, tiles, kblocks) ? 0.625 : 1.0);
}

template <int BN>
int32_t launch_igemm(mtl_ctx* ctx, const CUtensorMap* maps, const ConvTcParams& p) {
    using C = Cfg<BN>;
    auto kern = k_conv_igemm<BN>;
    MTL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    int tiles = p.tiles_w * p.tiles_h * p.tiles_nb * p.tiles_k;
    int grid = tiles < ctx->sm_count ? tiles : ctx->sm_count;
    {
        mtl_prof_scope prof(ctx, MTL_PROF_CONV_IGEMM);
        mtl_launch_pdl(ctx, kern, dim3(grid), dim3(kThreads), (size_t)(C::kSmemBytes), maps[0], maps[1], maps[2], maps[3], p);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

bool igemm_channel_major(const IgemmCall& c) {
    return c.Kout > 32 && (int64_t)c.N * c.OH * c.OW >= 1024 && (int64_t)c.N * c.Kout * c.OH * c.OW < (1ll << 31) &&
           mtl_global_tuning().conv_channel_major;
}
// Two taps per instruction when the layer has at most 64 output channels (see ConvTParams::paired).
bool igemm_paired(const IgemmCall& c, int x3) {
    // Pairing shortens the main loop but lengthens the epilogue (a second TMEM read per column chunk): it
    // pays only when the reduction per tile is long enough for the main loop to be the longer of the two.
    // A 3xTF32 k-block issues three products, so its main loop is three times as long.
    const int paired_kblocks = c.R * ((c.S + 1) / 2) * ((c.Cin + 31) / 32) * (x3 ? 3 : 1);
    return igemm_channel_major(c) && c.Kout <= 64 && c.S >= 2 && c.OW + 1 <= 240 &&
           paired_kblocks >= mtl_global_tuning().conv_paired_min_kblocks && mtl_global_tuning().conv_paired;
}
// At most 64 output channels without pairing: the channels are still spread over the four TMEM lane
// quadrants (16 each) so that all four epilogue warps store, instead of two doing all of it.
bool igemm_spread(const IgemmCall& c, int x3) {
    return igemm_channel_major(c) && c.Kout <= 64 && !igemm_paired(c, x3) &&
           mtl_global_tuning().conv_spread;
}
// Floats of one re-laid-out copy of the weights.
size_t igemm_weight_floats(const IgemmCall& c, int x3) {
    const size_t plain = (size_t)c.wK * c.wC * c.R * c.S;
    if (igemm_paired(c, x3)) return (size_t)c.R * ((c.S + 1) / 2) * 128 * c.Cin;
    if (igemm_spread(c, x3)) return (size_t)c.R * c.S * 128 * c.Cin;
    return plain;
}

// Channels-last copy (hi [, lo]) of an NCHW tensor; see k_nchw_to_nhwc for `colsum`.
int32_t stage_nhwc(mtl_ctx* ctx, float* hi, float* lo, const float* src, int N, int C, int HW, int x3, float* colsum) {
    dim3 tg((unsigned)((HW + 31) / 32), (unsigned)((C + 31) / 32), (unsigned)N);
    MTL_REQUIRE(ctx, N <= 65535 && tg.y <= 65535u, "batch too large for the layout pass");
    if (x3) mtl_launch_pdl(ctx, k_nchw_to_nhwc<true>, dim3(tg), dim3(256), (size_t)(0), hi, lo, src, C, HW, colsum);
    else mtl_launch_pdl(ctx, k_nchw_to_nhwc<false>, dim3(tg), dim3(256), (size_t)(0), hi, lo, src, C, HW, colsum);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t run_igemm_core(mtl_ctx* ctx, const IgemmCall& c, int x3, float* a_hi, float* a_lo, float* w_hi, float* w_lo);

int32_t run_igemm(mtl_ctx* ctx, const IgemmCall& c, int x3) {
    const int HW = c.IH * c.IW;
    const size_t n_act = (size_t)c.N * c.Cin * HW;
    const size_t n_wt = igemm_weight_floats(c, x3);
    const size_t act_pad = (n_act + 63) & ~(size_t)63, wt_pad = (n_wt + 63) & ~(size_t)63;
    const int parts = x3 ? 2 : 1;
    void* ws;
    if (c.act_cl && !x3) {
        // the caller keeps a channels-last copy of the activations: only the weights need scratch
        int32_t rc0 = mtl_workspace(ctx, wt_pad * 4, &ws);
        if (rc0) return rc0;
        return run_igemm_core(ctx, c, x3, const_cast<float*>(c.act_cl), nullptr, (float*)ws, nullptr);
    }
    int32_t rc = mtl_workspace(ctx, (size_t)parts * (act_pad + wt_pad) * 4, &ws);
    if (rc) return rc;
    float* a_hi = (float*)ws;
    float* a_lo = x3 ? a_hi + act_pad : nullptr;
    float* w_hi = a_hi + (size_t)parts * act_pad;
    float* w_lo = x3 ? w_hi + wt_pad : nullptr;

    dim3 tgrid((unsigned)((HW + 31) / 32), (unsigned)((c.Cin + 31) / 32), (unsigned)c.N);
    MTL_REQUIRE(ctx, c.N <= 65535 && tgrid.y <= 65535u, "batch too large for the layout pass");
    if (x3) mtl_launch_pdl(ctx, k_nchw_to_nhwc<true>, dim3(tgrid), dim3(256), (size_t)(0), a_hi, a_lo, c.act, c.Cin, HW, nullptr);
    else mtl_launch_pdl(ctx, k_nchw_to_nhwc<false>, dim3(tgrid), dim3(256), (size_t)(0), a_hi, a_lo, c.act, c.Cin, HW, nullptr);
    MTL_LAUNCHED(ctx);
    return run_igemm_core(ctx, c, x3, a_hi, a_lo, w_hi, w_lo);
}

// Weight re-layout and the implicit-GEMM kernel; the channels-last activations are already in place.
int32_t run_igemm_core(mtl_ctx* ctx, const IgemmCall& c, int x3, float* a_hi, float* a_lo, float* w_hi, float* w_lo) {
    const size_t n_wt = igemm_weight_floats(c, x3);
    int32_t rc = MTL_OK;
    const bool channel_major = igemm_channel_major(c);
    const bool paired = igemm_paired(c, x3);
    const bool spread = igemm_spread(c, x3);
    int wgrid = mtl_grid_for((int64_t)n_wt, 256, ctx->sm_count, 8);
    if (paired || spread) {
        if (x3) mtl_launch_pdl(ctx, k_weights_relayout_paired<true>, dim3(wgrid), dim3(256), (size_t)(0), w_hi, w_lo, c.wt, c.wK, c.wC, c.R, c.S, c.flip, paired ? 1 : 0);
        else mtl_launch_pdl(ctx, k_weights_relayout_paired<false>, dim3(wgrid), dim3(256), (size_t)(0), w_hi, w_lo, c.wt, c.wK, c.wC, c.R, c.S, c.flip, paired ? 1 : 0);
    } else {
        if (x3) mtl_launch_pdl(ctx, k_weights_relayout<true>, dim3(wgrid), dim3(256), (size_t)(0), w_hi, w_lo, c.wt, c.wK, c.wC, c.R, c.S, c.flip);
        else mtl_launch_pdl(ctx, k_weights_relayout<false>, dim3(wgrid), dim3(256), (size_t)(0), w_hi, w_lo, c.wt, c.wK, c.wC, c.R, c.S, c.flip);
    }
    MTL_LAUNCHED(ctx);

    if (channel_major) {
        ConvTParams q;
        q.N = c.N; q.OH = c.OH; q.OW = c.OW; q.Kout = c.Kout; q.Cin = c.Cin;
        q.R = c.R; q.S = c.S; q.ph = c.ph; q.pw = c.pw;
        q.paired = paired ? 1 : (spread ? 2 : 0);
        q.s_count = paired ? (c.S + 1) / 2 : c.S;
        q.s_step = paired ? 2 : 1;
        q.acc_stride = paired ? 248 : 256;
        q.pool = c.pool;
        q.pool_idx = c.pool_idx;
        const int kblocks = c.R * q.s_count * ((c.Cin + BK - 1) / BK) * (x3 ? 3 : 1);
        if (c.pool) {
            // whole rows, two of them, as many images as fit while the last 32-column read stays inside
            q.bw = c.OW;
            q.bh = 2;
            int bn_max = (256 - 32) / (2 * c.OW) + 1;
            if (bn_max > c.N) bn_max = c.N;
            // images per box: fewest (waves of tiles) x (TMA rows and boxes of a k-block), which for a small
            // batch is not always the fullest box (two waves of shorter tiles beat two waves of full ones)
            double best = 1e30;
            q.bn = bn_max;
            for (int bn = bn_max; bn >= 1; --bn) {
                const int64_t tiles = (int64_t)(c.OH / 2) * ((c.N + bn - 1) / bn) * ((c.Kout + BM - 1) / BM);
                const double cost = igemm_waves(ctx, tiles, kblocks) * (128 + 2 * c.OW * bn + 70);
                if (cost < best * 0.98) { best = cost; q.bn = bn; }
            }
        } else if (paired) {
            // whole rows plus the extra column; the box that fills most of 240 columns.  When the rows are a
            // multiple of four pixels wide the box is widened to the next multiple of four, so that every
            // group of four accumulator columns is either four aligned pixels of one row (one 16-byte store)
            // or entirely outside the image
            q.bw = (c.OW % 4 == 0 && c.OW + 4 <= 240) ? c.OW + 4 : c.OW + 1;
            double best = -1.0;
            for (int bh = 1; bh <= c.OH && q.bw * bh <= 240; ++bh) {
                int bn = 240 / (q.bw * bh);
                if (bn > c.N) bn = c.N;
                int64_t tiles = (int64_t)((c.OH + bh - 1) / bh) * ((c.N + bn - 1) / bn);
                double eff = (double)c.OW * c.OH * c.N / ((double)tiles * 240.0) + 1e-4 * bh;
                if (eff > best) { best = eff; q.bh = bh; q.bn = bn; }
            }
            // then fewer images per box if that shortens (waves of tiles) x (TMA rows and boxes of a
            // k-block): for a small batch two waves of shorter tiles beat two waves of full ones
            double cost0 = 1e30;
            for (int bn = q.bn, bn0 = q.bn; bn >= 1; --bn) {
                const int64_t tiles = (int64_t)((c.OH + q.bh - 1) / q.bh) * ((c.N + bn - 1) / bn);
                const double cost = igemm_waves(ctx, tiles, kblocks) * (128 + q.bw * q.bh * bn + 70);
                if (bn == bn0) cost0 = cost;
                if (cost < cost0 * 0.98) { cost0 = cost; q.bn = bn; }
            }
        } else {
            choose_box_n(c.OW, c.OH, c.N, 256, &q.bw, &q.bh, &q.bn);
        }
        q.npix = q.bw * q.bh * q.bn;
        q.n_mma = (q.npix + 15) / 16 * 16;
        q.tiles_w = (c.OW + q.bw - 1) / q.bw;
        q.tiles_h = (c.OH + q.bh - 1) / q.bh;
        q.tiles_nb = (c.N + q.bn - 1) / q.bn;
        q.tiles_k = (c.Kout + BM - 1) / BM;
        q.nseg = x3 ? 3 : 1;
        // segA selects the activation map, segB the weight map: lo*hi, hi*lo, hi*hi
        if (x3) { q.segA[0] = 1; q.segB[0] = 0; q.segA[1] = 0; q.segB[1] = 1; q.segA[2] = 0; q.segB[2] = 0; }
        else    { q.segA[0] = q.segA[1] = q.segA[2] = 0; q.segB[0] = q.segB[1] = q.segB[2] = 0; }
        q.out = c.out; q.bias = c.bias; q.accumulate = c.accumulate; q.relu = c.relu; q.status = ctx->dev_status;
        q.vec_ok = ((c.OH * c.OW) % 4 == 0) && ((reinterpret_cast<uintptr_t>(c.out) & 15) == 0);
        CUtensorMap tm[4];
        for (int i = 0; i < 2; ++i) {
            const float* a = (i == 1 && x3) ? a_lo : a_hi;
            const float* w = (i == 1 && x3) ? w_lo : w_hi;
            uint64_t adims[4] = {(uint64_t)c.Cin, (uint64_t)c.IW, (uint64_t)c.IH, (uint64_t)c.N};
            uint64_t astr[3] = {(uint64_t)c.Cin * 4, (uint64_t)c.IW * c.Cin * 4, (uint64_t)c.IH * c.IW * c.Cin * 4};
            uint32_t abox[4] = {BK, (uint32_t)q.bw, (uint32_t)q.bh, (uint32_t)q.bn};
            rc = mtl_encode_tmap(ctx, &tm[i], a, 4, adims, astr, abox);
            if (rc) return rc;
            const uint64_t wrows = (paired || spread) ? 128 : (uint64_t)c.Kout;
            uint64_t wdims[3] = {(uint64_t)c.Cin, wrows, (uint64_t)(c.R * q.s_count)};
            uint64_t wstr[2] = {(uint64_t)c.Cin * 4, wrows * c.Cin * 4};
            uint32_t wbox[3] = {BK, (uint32_t)BM, 1};
            rc = mtl_encode_tmap(ctx, &tm[2 + i], w, 3, wdims, wstr, wbox);
            if (rc) return rc;
        }
        MTL_CUDA(ctx, cudaFuncSetAttribute(k_conv_igemm_t, cudaFuncAttributeMaxDynamicSharedMemorySize, kTSmemBytes));
        const int tiles = q.tiles_w * q.tiles_h * q.tiles_nb * q.tiles_k;
        q.whole_items = q.n_items = tiles;
        q.kb_half = 0;
        q.split_scratch = nullptr;
        q.split_tickets = ctx->tickets + 4096;
        if (igemm_tail_splits(ctx, tiles, kblocks)) {
            const int rem = tiles % ctx->sm_count;   // 2 * rem <= sm_count <= sm_count_total slots of scratch
            void* sp;
            rc = mtl_split_scratch(ctx, &sp);
            if (rc) return rc;
            q.split_scratch = (float4*)sp;
            q.whole_items = tiles - rem;
            q.n_items = q.whole_items + 2 * rem;
            q.kb_half = (kblocks + 1) / 2;
            ctx->conv_split_tiles += rem;
        }
        int grid = q.n_items < ctx->sm_count ? q.n_items : ctx->sm_count;
        {
            mtl_prof_scope prof(ctx, MTL_PROF_CONV_IGEMM);
            mtl_launch_pdl(ctx, k_conv_igemm_t, dim3(grid), dim3(kThreads), (size_t)(kTSmemBytes), tm[0], tm[1], tm[2], tm[3], q);
        }
        MTL_LAUNCHED(ctx);
        return MTL_OK;
    }

    ConvTcParams p;
    p.N = c.N; p.OH = c.OH; p.OW = c.OW; p.Kout = c.Kout; p.Cin = c.Cin;
    p.R = c.R; p.S = c.S; p.ph = c.ph; p.pw = c.pw;
    choose_box(c.OW, c.OH, c.N, &p.bw, &p.bh, &p.bn);
    p.tiles_w = (c.OW + p.bw - 1) / p.bw;
    p.tiles_h = (c.OH + p.bh - 1) / p.bh;
    p.tiles_nb = (c.N + p.bn - 1) / p.bn;
    const int BN = c.Kout > 64 ? 128 : 64;
    p.tiles_k = (c.Kout + BN - 1) / BN;
    p.nseg = x3 ? 3 : 1;
    if (x3) { p.segA[0] = 1; p.segB[0] = 0; p.segA[1] = 0; p.segB[1] = 1; p.segA[2] = 0; p.segB[2] = 0; }
    else    { p.segA[0] = p.segA[1] = p.segA[2] = 0; p.segB[0] = p.segB[1] = p.segB[2] = 0; }
    p.a_bytes = (uint32_t)(p.bw * p.bh * p.bn) * 128u;
    p.out = c.out; p.bias = c.bias; p.accumulate = c.accumulate; p.status = ctx->dev_status;

    CUtensorMap maps[4];
    for (int i = 0; i < 2; ++i) {
        const float* a = (i == 1 && x3) ? a_lo : a_hi;
        const float* w = (i == 1 && x3) ? w_lo : w_hi;
        uint64_t adims[4] = {(uint64_t)c.Cin, (uint64_t)c.IW, (uint64_t)c.IH, (uint64_t)c.N};
        uint64_t astr[3] = {(uint64_t)c.Cin * 4, (uint64_t)c.IW * c.Cin * 4, (uint64_t)c.IH * c.IW * c.Cin * 4};
        uint32_t abox[4] = {BK, (uint32_t)p.bw, (uint32_t)p.bh, (uint32_t)p.bn};
        rc = mtl_encode_tmap(ctx, &maps[i], a, 4, adims, astr, abox);
        if (rc) return rc;
        uint64_t wdims[3] = {(uint64_t)c.Cin, (uint64_t)c.Kout, (uint64_t)(c.R * c.S)};
        uint64_t wstr[2] = {(uint64_t)c.Cin * 4, (uint64_t)c.Kout * c.Cin * 4};
        uint32_t wbox[3] = {BK, (uint32_t)BN, 1};
        rc = mtl_encode_tmap(ctx, &maps[2 + i], w, 3, wdims, wstr, wbox);
        if (rc) return rc;
    }
    rc = (BN == 128) ? launch_igemm<128>(ctx, maps, p) : launch_igemm<64>(ctx, maps, p);
    if (rc) return rc;
    if (c.relu)  // this kernel has no fused activation: one in-place pass over the result
        return mtl_unary_fwd(ctx, MTL_OP_RELU, c.out, c.out, (int64_t)c.N * c.Kout * c.OH * c.OW, 0.0f, 0.0f);
    return MTL_OK;
}

bool igemm_geometry_ok(const ConvGeom& g) {
    return g.sh == 1 && g.sw == 1 && g.dh == 1 && g.dw == 1;
}

// ------------------------------------------------------------------ kernel gradient -----------
// dW[k, c, r, s] = sum over pixels (n, oh, ow) of ug[n, k, oh, ow] * X[n, c, oh + r - ph, ow + s - pw].
// GEMM view per filter tap: D_tap[k, c] with the pixels as the reduction axis.  Both operands are
// channels-last copies, so the channel axis (k of ug, c of X) is contiguous = MN-major tiles:
//   A  {128 out-channels x 32 pixels}  from ug,  one TMA box {32 ch, bw, bh, bn} per 32 channels
//   B  {C in-channels x 32 pixels} per tap, from X, box origin shifted by the tap, zero fill = padding
// One CTA owns a group of T taps (T*C <= 512 accumulator columns), one 128-wide slice of the
// output channels and a contiguous range of pixel chunks; the A tile of a stage is shared by all
// taps of the group.  Partial sums go to scratch [split][tap][k][c] and are folded by a second
// kernel in a fixed order (deterministic).

constexpr int kWgradPix = 32;  // pixels per pipeline stage = reduction extent of 4 MMAs

struct WgradParams {
    int N, OH, OW, Kout, C;
    int R, S, ph, pw;
    int bw, bh, bn;             // pixel box, bw*bh*bn == 32
    int tiles_w, tiles_h, tiles_nb;
    int T, ngroups, ktiles, nsplit, chunks_per_split;
    int stages, stage_bytes;
    int nseg, segA[3], segB[3];
    uint32_t tmem_cols;
    float* partial;             // [nsplit][R*S][Kout][C]
    int32_t* status;
};

__global__ void __launch_bounds__(kThreads, 1)
k_conv_wgrad_tc(const __grid_constant__ CUtensorMap mapU0, const __grid_constant__ CUtensorMap mapU1,
                const __grid_constant__ CUtensorMap mapX0, const __grid_constant__ CUtensorMap mapX1, WgradParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.stages * p.stage_bytes);
    uint64_t* full = bars;
    uint64_t* empty = bars + 8;
    uint64_t* acc_full = bars + 16;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // work item: (tap group, out-channel tile, pixel split)
    int item = blockIdx.x;
    const int split = item % p.nsplit;
    item /= p.nsplit;
    const int kt = item % p.ktiles;
    const int grp = item / p.ktiles;
    const int tap0 = grp * p.T;
    const int ntaps = min(p.T, p.R * p.S - tap0);
    const int cchunks = p.C / 32;
    const int total_chunks = p.tiles_w * p.tiles_h * p.tiles_nb;
    const int chunk_begin = split * p.chunks_per_split;
    const int chunk_end = min(total_chunks, chunk_begin + p.chunks_per_split);
    const int n_chunks = max(0, chunk_end - chunk_begin);
    const int kb_total = n_chunks * p.nseg;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&mapU0);
        prefetch_tensormap(&mapX0);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, p.tmem_cols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    mtl_pdl_sync();   // everything above touched only shared / tensor memory
    const uint32_t a_bytes = 4u * 4096u;
    const uint32_t tx_bytes = a_bytes + (uint32_t)(ntaps * cchunks) * 4096u;

    if (warp == 0) {
        // The whole warp produces: issuing a TMA copy costs its thread a few hundred cycles, so the
        // operand boxes of one stage are issued by different lanes at once (lane 0: the ug tile and
        // the byte count, lane 1 + t: the input box of tap t).
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int kb = 0; kb < kb_total; ++kb) {
            if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, kWaitBudgetNs)) ok = false;
            if (__any_sync(0xffffffffu, !ok)) { ok = false; break; }
            const int seg = kb / n_chunks;
            int pc = chunk_begin + (kb - seg * n_chunks);
            const int tw = pc % p.tiles_w;
            pc /= p.tiles_w;
            const int th = pc % p.tiles_h;
            const int tnb = pc / p.tiles_h;
            const int ow0 = tw * p.bw, oh0 = th * p.bh, n0 = tnb * p.bn;
            const CUtensorMap* mu = p.segA[seg] ? &mapU1 : &mapU0;
            const CUtensorMap* mx = p.segB[seg] ? &mapX1 : &mapX0;
            uint8_t* sa = tiles + stage * p.stage_bytes;
            uint8_t* sb = sa + a_bytes;
            if (lane == 0) mbar_arrive_expect_tx(&full[stage], tx_bytes);
            __syncwarp();
            // one 5-D box per operand tile {32 channels, bw, bh, bn pixels, channel chunks}: the TMA
            // unit spends about 35 ns per box besides about 1 ns per 128-byte row, so boxes stay large
            if (lane == 0) {
                tma_load_5d(sa, mu, &full[stage], 0, ow0, oh0, n0, kt * (BM / 32));
            } else if (lane <= ntaps) {
                const int t = lane - 1;
                const int rs = tap0 + t;
                const int r = rs / p.S, s = rs - r * p.S;
                tma_load_5d(sb + t * cchunks * 4096, mx, &full[stage], 0, ow0 + s - p.pw, oh0 + r - p.ph, n0, 0);
            }
            if (++stage == p.stages) { stage = 0; phase ^= 1u; }
        }
        if (!ok && lane == 0) atomicExch(p.status, MTL_ERR_TIMEOUT);
    } else if (warp == 1) {
        if (lane == 0) {
            // taps are multiplied in groups of up to 256 / C so that one instruction covers several
            const int taps_per_mma = max(1, 256 / p.C);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < kb_total && ok; ++kb) {
                if (!mbar_wait(&full[stage], phase, abort_flag, kWaitBudgetNs)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(tiles + stage * p.stage_bytes);
                const uint32_t sb = sa + a_bytes;
                for (int t0 = 0; t0 < ntaps; t0 += taps_per_mma) {
                    const int nt = min(taps_per_mma, ntaps - t0);
                    const uint32_t idesc = make_idesc_tf32(nt * p.C, true, true);
                    const uint32_t sbt = sb + (uint32_t)(t0 * cchunks) * 4096u;
#pragma unroll
                    for (int kk = 0; kk < kWgradPix / 8; ++kk)
                        mma_tf32(tmem_base + (uint32_t)(t0 * p.C), desc_mn_major(sa, kk), desc_mn_major(sbt, kk), idesc,
                                 (kb | kk) ? 1u : 0u);
                }
                mma_commit(&empty[stage]);
                if (++stage == p.stages) { stage = 0; phase ^= 1u; }
            }
            if (ok) mma_commit(acc_full);
            else atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else {
        const int quad = warp & 3;
        const int k = kt * BM + quad * 32 + lane;
        bool ok = true;
        if (kb_total > 0) {
            ok = mbar_wait(acc_full, 0, abort_flag, kWaitBudgetNs);
            tc_fence_after_sync();
        }
        if (ok) {
            for (int t = 0; t < ntaps; ++t) {
                float* dst = p.partial + (((int64_t)split * p.R * p.S + tap0 + t) * p.Kout + k) * p.C;
                for (int jc = 0; jc < cchunks; ++jc) {
                    uint32_t r[32];
                    if (kb_total > 0) {
                        tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(t * p.C + jc * 32), r);
                        tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = 0u;
                    }
                    if (k < p.Kout) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<float4*>(dst + jc * 32 + j) =
                                make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]),
                                            __uint_as_float(r[j + 3]));
                    }
                }
            }
        } else if (lane == 0) {
            atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, p.tmem_cols);
    }
}

// dW[k][c][r][s] (+)= sum over splits of partial[split][rs][k][c]
// Column sums of a [rows, cols] matrix of per-block channel sums (the bias gradient), run by the extra blocks
// of the fold launch below: a block owns eight columns, its 32 row lanes walk the rows 32 apart with sixteen
// loads in flight and meet in shared memory, lane 0 first -- a fixed order whatever the grid.
struct BiasFold {
    float* db = nullptr;          // null: no bias gradient in this launch
    const float* part = nullptr;
    int64_t rows = 0;
    int cols = 0;
    int accumulate = 0;
};
__device__ void bias_fold_block(const BiasFold& b, int blk) {
    __shared__ float part[32][9];
    const int cl = threadIdx.x & 7, rl = threadIdx.x >> 3;
    const int c = blk * 8 + cl;
    float s = 0.0f;
    if (c < b.cols) {
        int64_t r = rl;
        for (; r + 15 * 32 < b.rows; r += 16 * 32) {
            float a[16];
#pragma unroll
            for (int u = 0; u < 16; ++u) a[u] = b.part[(r + 32 * u) * b.cols + c];
#pragma unroll
            for (int u = 0; u < 16; ++u) s += a[u];
        }
        for (; r < b.rows; r += 32) s += b.part[r * b.cols + c];
    }
    part[rl][cl] = s;
    __syncthreads();
    if (rl == 0 && c < b.cols) {
        float t = 0.0f;
#pragma unroll
        for (int j = 0; j < 32; ++j) t += part[j][cl];
        b.db[c] = b.accumulate ? b.db[c] + t : t;
    }
}

__global__ void __launch_bounds__(256) k_wgrad_fold(float* __restrict__ dW, const float* __restrict__ partial, int K,
                                                    int C, int RS, int nsplit, int accumulate, int fold_blocks, BiasFold bias) {
    mtl_pdl_sync();
    if ((int)blockIdx.x >= fold_blocks) {
        bias_fold_block(bias, (int)blockIdx.x - fold_blocks);
        return;
    }
    const int64_t total = (int64_t)K * C * RS;
    if ((C & 3) == 0) {
        // four channels per thread: 16-byte loads of the partials, eight slices in flight, slices added in
        // ascending order
        const int64_t total4 = total >> 2;
        const float4* p4 = reinterpret_cast<const float4*>(partial);
        for (int64_t i4 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i4 < total4; i4 += (int64_t)fold_blocks * blockDim.x) {
            const int64_t i = i4 << 2;             // scratch layout [rs][k][c]
            const int c = (int)(i % C);
            const int64_t q = i / C;
            const int k = (int)(q % K);
            const int rs = (int)(q / K);
            float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            int j = 0;
            for (; j + 8 <= nsplit; j += 8) {
                float4 t[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) t[u] = p4[(int64_t)(j + u) * total4 + i4];
#pragma unroll
                for (int u = 0; u < 8; ++u) { s.x += t[u].x; s.y += t[u].y; s.z += t[u].z; s.w += t[u].w; }
            }
            for (; j < nsplit; ++j) {
                const float4 t = p4[(int64_t)j * total4 + i4];
                s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
            }
            float* o = dW + ((int64_t)k * C + c) * RS + rs;
            if (accumulate) { o[0] += s.x; o[RS] += s.y; o[2 * RS] += s.z; o[3 * RS] += s.w; }
            else { o[0] = s.x; o[RS] = s.y; o[2 * RS] = s.z; o[3 * RS] = s.w; }
        }
        return;
    }
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)fold_blocks * blockDim.x;
    for (int64_t i = tid; i < total; i += stride) {
        // i enumerates the scratch layout [rs][k][c] so that reads are coalesced
        int c = (int)(i % C);
        int64_t q = i / C;
        int k = (int)(q % K);
        int rs = (int)(q / K);
        // eight partials in flight at a time, added in ascending order (the loads do not depend on one another)
        float s = 0.0f;
        int j = 0;
        for (; j + 8 <= nsplit; j += 8) {
            float t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) t[u] = partial[(int64_t)(j + u) * total + i];
#pragma unroll
            for (int u = 0; u < 8; ++u) s += t[u];
        }
        for (; j < nsplit; ++j) s += partial[(int64_t)j * total + i];
        int64_t o = ((int64_t)k * C + c) * RS + rs;
        dW[o] = accumulate ? dW[o] + s : s;
    }
}

// A 32-pixel box {bw, bh, bn} (powers of two) covering the output with the least overhang.
void choose_box32(int OW, int OH, int N, int* bw_, int* bh_, int* bn_) {
    double best = -1.0;
    for (int bw = 1; bw <= 32; bw *= 2)
        for (int bh = 1; bw * bh <= 32; bh *= 2) {
            int bn = 32 / (bw * bh);
            int64_t tiles = (int64_t)((OW + bw - 1) / bw) * ((OH + bh - 1) / bh) * ((N + bn - 1) / bn);
            double eff = (double)OW * OH * N / ((double)tiles * 32.0) + 1e-4 * bw;
            if (eff > best) { best = eff; *bw_ = bw; *bh_ = bh; *bn_ = bn; }
        }
}

}  // namespace

bool mtl_conv_fwd_tc_supported(const ConvGeom& g, const float* X, const float* Wt, const float* Y) {
    if (!igemm_geometry_ok(g)) return false;
    if (g.C < 16 || (g.C % 4) || g.K < 16) return false;
    if ((int64_t)g.N * g.OH * g.OW < 128) return false;
    if ((((uintptr_t)X) | ((uintptr_t)Wt) | ((uintptr_t)Y)) & 15u) return false;
    return true;
}

bool mtl_conv_dgrad_tc_supported(const ConvGeom& g, const float* ug, const float* Wt, const float* dX) {
    if (!igemm_geometry_ok(g)) return false;
    if (g.K < 16 || (g.K % 4) || g.C < 16) return false;
    if ((int64_t)g.N * g.H * g.W < 128) return false;
    if (g.ph > g.R - 1 || g.pw > g.S - 1) return false;
    if ((((uintptr_t)ug) | ((uintptr_t)Wt) | ((uintptr_t)dX)) & 15u) return false;
    return true;
}

// CONV2D (+ RELU) + 2x2 / stride-2 MAXPOOL2D in the epilogue of the channel-major kernel.
bool mtl_conv_fwd_pool_tc_supported(const ConvGeom& g, const float* X, const float* Wt, const float* pooled) {
    if (!mtl_conv_fwd_tc_supported(g, X, Wt, pooled)) return false;
    IgemmCall c;
    c.N = g.N; c.Cin = g.C; c.IH = g.H; c.IW = g.W; c.Kout = g.K; c.OH = g.OH; c.OW = g.OW;
    c.R = g.R; c.S = g.S; c.ph = g.ph; c.pw = g.pw; c.wK = g.K; c.wC = g.C; c.flip = 0;
    return igemm_channel_major(c) && g.K > 64 && g.OW % 2 == 0 && g.OW <= 16 && g.OH % 2 == 0 &&
           mtl_global_tuning().conv_pool_epilogue;
}

int32_t mtl_conv_fwd_pool_tc(mtl_ctx* ctx, float* pooled, int32_t* idx, const float* X, const float* Wt,
                             const float* bias, const ConvGeom& g, int x3, int relu, const float* X_cl) {
    IgemmCall c;
    c.N = g.N; c.Cin = g.C; c.IH = g.H; c.IW = g.W; c.Kout = g.K; c.OH = g.OH; c.OW = g.OW;
    c.R = g.R; c.S = g.S; c.ph = g.ph; c.pw = g.pw;
    c.act = X; c.wt = Wt; c.wK = g.K; c.wC = g.C; c.flip = 0;
    c.out = pooled; c.bias = bias; c.accumulate = 0; c.relu = relu; c.act_cl = X_cl;
    c.pool = 1; c.pool_idx = idx;
    return run_igemm(ctx, c, x3);
}

// Plain channels-last copy [N, C, HW] -> [N, HW, C] (no operand split), for callers that keep one.
int32_t mtl_channels_last_copy(mtl_ctx* ctx, float* dst, const float* src, int N, int C, int HW) {
    return stage_nhwc(ctx, dst, nullptr, src, N, C, HW, 0, nullptr);
}

int32_t mtl_conv_fwd_tc(mtl_ctx* ctx, float* Y, const float* X, const float* Wt, const float* bias,
                        const ConvGeom& g, int x3, int relu, const float* X_cl) {
    IgemmCall c;
    c.N = g.N; c.Cin = g.C; c.IH = g.H; c.IW = g.W; c.Kout = g.K; c.OH = g.OH; c.OW = g.OW;
    c.R = g.R; c.S = g.S; c.ph = g.ph; c.pw = g.pw;
    c.act = X; c.wt = Wt; c.wK = g.K; c.wC = g.C; c.flip = 0;
    c.out = Y; c.bias = bias; c.accumulate = 0; c.relu = relu; c.act_cl = X_cl;
    return run_igemm(ctx, c, x3);
}

int32_t mtl_conv_dgrad_tc(mtl_ctx* ctx, float* dX, const float* ug, const float* Wt, const ConvGeom& g,
                          int accumulate, int x3) {
    IgemmCall c;
    c.N = g.N; c.Cin = g.K; c.IH = g.OH; c.IW = g.OW; c.Kout = g.C; c.OH = g.H; c.OW = g.W;
    c.R = g.R; c.S = g.S; c.ph = g.R - 1 - g.ph; c.pw = g.S - 1 - g.pw;
    c.act = ug; c.wt = Wt; c.wK = g.K; c.wC = g.C; c.flip = 1;
    c.out = dX; c.bias = nullptr; c.accumulate = accumulate; c.relu = 0;
    return run_igemm(ctx, c, x3);
}

bool mtl_conv_wgrad_tc_supported(const ConvGeom& g, const float* ug, const float* X, const float* dW) {
    if (!igemm_geometry_ok(g)) return false;
    if (g.C < 32 || (g.C % 32) || g.C > 256 || g.K < 32 || (g.K % 32)) return false;
    if ((int64_t)g.N * g.OH * g.OW < 4096) return false;  // too little reduction work to split
    if ((((uintptr_t)ug) | ((uintptr_t)X) | ((uintptr_t)dW)) & 15u) return false;
    return true;
}

namespace {

// Geometry of the kernel-gradient launch; the number of floats of partial sums it needs.
int32_t wgrad_plan(mtl_ctx* ctx, const ConvGeom& g, int x3, WgradParams* pp, size_t* n_part) {
    WgradParams& p = *pp;
    p.N = g.N; p.OH = g.OH; p.OW = g.OW; p.Kout = g.K; p.C = g.C;
    p.R = g.R; p.S = g.S; p.ph = g.ph; p.pw = g.pw;
    choose_box32(g.OW, g.OH, g.N, &p.bw, &p.bh, &p.bn);
    p.tiles_w = (g.OW + p.bw - 1) / p.bw;
    p.tiles_h = (g.OH + p.bh - 1) / p.bh;
    p.tiles_nb = (g.N + p.bn - 1) / p.bn;
    const int RS = g.R * g.S;
    // taps per CTA: fit the accumulator columns, then balance the groups
    int tmax = 512 / g.C;
    if (tmax > RS) tmax = RS;
    // The kernel is bound by filling shared memory from L2 (every tap re-reads its shifted input box), not
    // by the tensor pipe: measured on the 64->128 channel 5x5 layer, t = 4, 5, 6, 7, 8 taps per CTA take
    // 0.384, 0.299, 0.317, 0.274, 0.353 ms.  Modelled time of a CTA: (bytes of one stage + a fixed 16 KB
    // worth of per-stage overhead) x (pixel chunks per CTA); the CTAs left after dividing the SMs by the tap
    // groups split the pixels, and at least three stages must fit shared memory.  Every tap group gets
    // the same number of CTAs even when the last group has fewer taps: groups that walk the pixels in
    // step share the gradient tiles in L2, groups at different speeds fetch them from DRAM once each
    // (measured: 0.307 ms with the SMs shared out by work, 0.274 ms with equal shares).
    int best_t = 1;
    double best_cost = 1e30;
    for (int t = 1; t <= tmax; ++t) {
        const int stage_bytes = 4 * 4096 + t * (g.C / 32) * 4096;
        if (t > 1 && (232448 - 2048) / stage_bytes < 3) break;
        const int groups = (RS + t - 1) / t;
        int ns = ctx->sm_count / (groups * ((g.K + BM - 1) / BM));
        if (ns < 1) ns = 1;
        const double cost = (double)(stage_bytes + 16384) / ns;
        if (cost < best_cost * 0.999) { best_cost = cost; best_t = t; }
    }
    if (ctx->tune.wgrad_taps >= 1 && ctx->tune.wgrad_taps <= tmax) best_t = ctx->tune.wgrad_taps;
    p.T = best_t;
    p.ngroups = (RS + p.T - 1) / p.T;
    p.ktiles = (g.K + BM - 1) / BM;
    const int total_chunks = p.tiles_w * p.tiles_h * p.tiles_nb;
    int nsplit = ctx->sm_count / (p.ngroups * p.ktiles);
    if (nsplit < 1) nsplit = 1;
    if (nsplit > total_chunks) nsplit = total_chunks;
    p.chunks_per_split = (total_chunks + nsplit - 1) / nsplit;
    p.nsplit = (total_chunks + p.chunks_per_split - 1) / p.chunks_per_split;
    p.stage_bytes = 4 * 4096 + p.T * (g.C / 32) * 4096;
    p.stages = (232448 - 2048) / p.stage_bytes;
    if (p.stages > 8) p.stages = 8;
    if (p.stages < 2) return mtl_set_error(ctx, MTL_ERR_UNSUPPORTED, "kernel-gradient tile does not fit shared memory");
    uint32_t cols = 32;
    while ((int)cols < p.T * g.C) cols *= 2;
    p.tmem_cols = cols;
    p.nseg = x3 ? 3 : 1;
    if (x3) { p.segA[0] = 1; p.segB[0] = 0; p.segA[1] = 0; p.segB[1] = 1; p.segA[2] = 0; p.segB[2] = 0; }
    else    { p.segA[0] = p.segA[1] = p.segA[2] = 0; p.segB[0] = p.segB[1] = p.segB[2] = 0; }
    p.status = ctx->dev_status;
    *n_part = (size_t)p.nsplit * RS * g.K * g.C;
    return MTL_OK;
}


// The launch itself: channels-last copies (hi [, lo]) of ug and X are in place.
int32_t wgrad_core(mtl_ctx* ctx, float* dW, const float* u_hi, const float* u_lo, const float* x_hi, const float* x_lo,
                   float* partial, WgradParams p, const ConvGeom& g, int accumulate, int x3, BiasFold bias = BiasFold()) {
    const int RS = g.R * g.S;
    int32_t rc = MTL_OK;
    p.partial = partial;
    CUtensorMap maps[4];
    for (int i = 0; i < 2; ++i) {
        const float* u = (i == 1 && x3) ? u_lo : u_hi;
        const float* x = (i == 1 && x3) ? x_lo : x_hi;
        // channels-last [N, H, W, Ch] viewed as {32, W, H, N, Ch/32}: the last axis steps 128 bytes
        uint32_t ubox[5] = {32, (uint32_t)p.bw, (uint32_t)p.bh, (uint32_t)p.bn, (uint32_t)(BM / 32)};
        uint64_t udims[5] = {32, (uint64_t)g.OW, (uint64_t)g.OH, (uint64_t)g.N, (uint64_t)(g.K / 32)};
        uint64_t ustr[4] = {(uint64_t)g.K * 4, (uint64_t)g.OW * g.K * 4, (uint64_t)g.OH * g.OW * g.K * 4, 128};
        rc = mtl_encode_tmap(ctx, &maps[i], u, 5, udims, ustr, ubox, true);
        if (rc) return rc;
        uint32_t xbox[5] = {32, (uint32_t)p.bw, (uint32_t)p.bh, (uint32_t)p.bn, (uint32_t)(g.C / 32)};
        uint64_t xdims[5] = {32, (uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.N, (uint64_t)(g.C / 32)};
        uint64_t xstr[4] = {(uint64_t)g.C * 4, (uint64_t)g.W * g.C * 4, (uint64_t)g.H * g.W * g.C * 4, 128};
        rc = mtl_encode_tmap(ctx, &maps[2 + i], x, 5, xdims, xstr, xbox, true);
        if (rc) return rc;
    }
    const int smem_bytes = p.stages * p.stage_bytes + 1024 + 256;
    MTL_CUDA(ctx, cudaFuncSetAttribute(k_conv_wgrad_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    const int grid = p.ngroups * p.ktiles * p.nsplit;
    {
        mtl_prof_scope prof(ctx, MTL_PROF_CONV_WGRAD);
        mtl_launch_pdl(ctx, k_conv_wgrad_tc, dim3(grid), dim3(kThreads), (size_t)(smem_bytes), maps[0], maps[1], maps[2], maps[3], p);
    }
    MTL_LAUNCHED(ctx);
    int fgrid = mtl_grid_for((int64_t)g.K * g.C * RS / ((g.C & 3) == 0 ? 4 : 1), 256, ctx->sm_count, 8);
    const int bias_blocks = bias.db ? (bias.cols + 7) / 8 : 0;
    mtl_launch_pdl(ctx, k_wgrad_fold, dim3(fgrid + bias_blocks), dim3(256), (size_t)(0), dW, p.partial, g.K, g.C, RS, p.nsplit, accumulate,
                   fgrid, bias);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

}  // namespace

int32_t mtl_conv_wgrad_tc(mtl_ctx* ctx, float* dW, const float* ug, const float* X, const ConvGeom& g,
                          int accumulate, int x3) {
    WgradParams p;
    size_t n_part;
    int32_t rc = wgrad_plan(ctx, g, x3, &p, &n_part);
    if (rc) return rc;
    // scratch: channels-last copies of ug and X (hi [, lo]) and the per-split partial sums
    const size_t n_u = (size_t)g.N * g.K * g.OH * g.OW, n_x = (size_t)g.N * g.C * g.H * g.W;
    const size_t u_pad = (n_u + 63) & ~(size_t)63, x_pad = (n_x + 63) & ~(size_t)63;
    const int parts = x3 ? 2 : 1;
    void* ws;
    rc = mtl_workspace(ctx, ((size_t)parts * (u_pad + x_pad) + n_part) * 4, &ws);
    if (rc) return rc;
    float* u_hi = (float*)ws;
    float* u_lo = x3 ? u_hi + u_pad : nullptr;
    float* x_hi = u_hi + (size_t)parts * u_pad;
    float* x_lo = x3 ? x_hi + x_pad : nullptr;
    float* partial = x_hi + (size_t)parts * x_pad;
    rc = stage_nhwc(ctx, u_hi, u_lo, ug, g.N, g.K, g.OH * g.OW, x3, nullptr);
    if (rc) return rc;
    rc = stage_nhwc(ctx, x_hi, x_lo, X, g.N, g.C, g.H * g.W, x3, nullptr);
    if (rc) return rc;
    return wgrad_core(ctx, dW, u_hi, u_lo, x_hi, x_lo, partial, p, g, accumulate, x3);
}

// dX, dW and (optionally) the bias gradient of one CONV2D from a single channels-last copy of ug:
// the kernel gradient runs first, then the input gradient re-uses the copy; the bias gradient is
// the per-channel sum the copy pass leaves behind.
int32_t mtl_conv_bwd_fused_tc(mtl_ctx* ctx, float* dX, float* dW, float* db, const float* ug, const float* X,
                              const float* Wt, const ConvGeom& g, int acc_dx, int acc_dw, int acc_db, int x3,
                              const float* X_cl) {
    return mtl_conv_bwd_fused_tc_src(ctx, dX, dW, db, ug, nullptr, nullptr, nullptr, 0, X, Wt, g, acc_dx, acc_dw, acc_db,
                                     x3, X_cl);
}

// The same with the upper gradient given either dense (ug) or pooled (pg, pidx, pv of a 2x2 / stride-2
// MAXPOOL2D behind an optional RELU): the pooled form is scattered straight into the channels-last copy.
int32_t mtl_conv_bwd_fused_tc_src(mtl_ctx* ctx, float* dX, float* dW, float* db, const float* ug, const float* pg,
                                  const int32_t* pidx, const float* pv, int relu, const float* X, const float* Wt,
                                  const ConvGeom& g, int acc_dx, int acc_dw, int acc_db, int x3, const float* X_cl) {
    WgradParams p;
    size_t n_part;
    int32_t rc = wgrad_plan(ctx, g, x3, &p, &n_part);
    if (rc) return rc;
    const size_t n_u = (size_t)g.N * g.K * g.OH * g.OW, n_x = (size_t)g.N * g.C * g.H * g.W;
    IgemmCall c;
    c.N = g.N; c.Cin = g.K; c.IH = g.OH; c.IW = g.OW; c.Kout = g.C; c.OH = g.H; c.OW = g.W;
    c.R = g.R; c.S = g.S; c.ph = g.R - 1 - g.ph; c.pw = g.S - 1 - g.pw;
    c.act = ug; c.wt = Wt; c.wK = g.K; c.wC = g.C; c.flip = 1;
    c.out = dX; c.bias = nullptr; c.accumulate = acc_dx; c.relu = 0;
    const size_t n_wt = igemm_weight_floats(c, x3);
    const size_t u_pad = (n_u + 63) & ~(size_t)63, x_pad = (n_x + 63) & ~(size_t)63, wt_pad = (n_wt + 63) & ~(size_t)63;
    const int parts = x3 ? 2 : 1;
    const int ptiles = pg ? 1 : (g.OH * g.OW + 31) / 32;  // rows of per-block channel sums per image
    const size_t n_bias = db ? ((size_t)g.N * ptiles + 256) * g.K : 0;
    size_t second = (size_t)parts * x_pad + n_part;
    if ((size_t)parts * wt_pad > second) second = (size_t)parts * wt_pad;
    void* ws;
    rc = mtl_workspace(ctx, ((size_t)parts * u_pad + second + n_bias) * 4, &ws);
    if (rc) return rc;
    float* u_hi = (float*)ws;
    float* u_lo = x3 ? u_hi + u_pad : nullptr;
    float* region = u_hi + (size_t)parts * u_pad;
    float* x_hi = region;
    float* x_lo = x3 ? x_hi + x_pad : nullptr;
    float* partial = region + (size_t)parts * x_pad;
    float* bias_part = region + second;
    if (pg) {
        const int POH = g.OH / 2, POW = g.OW / 2;
        const int PS = (POH * POW) | 1;
        const size_t smem = (size_t)2 * 32 * PS * 4;
        dim3 grid((unsigned)((g.K + 31) / 32), (unsigned)g.N);
        MTL_REQUIRE(ctx, g.N <= 65535 && smem <= 200 * 1024, "pooled plane too large for the scatter pass");
        if (x3) {
            MTL_CUDA(ctx, cudaFuncSetAttribute(k_pool_bwd_2x2_cl<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            mtl_launch_pdl(ctx, k_pool_bwd_2x2_cl<true>, dim3(grid), dim3(256), (size_t)(smem), u_hi, u_lo, db ? bias_part : nullptr, pg, pidx, pv, g.K, POH, POW, relu);
        } else {
            MTL_CUDA(ctx, cudaFuncSetAttribute(k_pool_bwd_2x2_cl<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            mtl_launch_pdl(ctx, k_pool_bwd_2x2_cl<false>, dim3(grid), dim3(256), (size_t)(smem), u_hi, u_lo, db ? bias_part : nullptr, pg, pidx, pv, g.K, POH, POW, relu);
        }
        MTL_LAUNCHED(ctx);
    } else {
        rc = stage_nhwc(ctx, u_hi, u_lo, ug, g.N, g.K, g.OH * g.OW, x3, db ? bias_part : nullptr);
        if (rc) return rc;
    }
    BiasFold bias_fold;
    if (db && (int64_t)g.N * ptiles <= 4096) {
        // few rows of per-block sums (the pooled path has one per image): summed by extra blocks of the
        // kernel-gradient fold launch instead of by launches of their own
        bias_fold.db = db; bias_fold.part = bias_part; bias_fold.rows = (int64_t)g.N * ptiles; bias_fold.cols = g.K;
        bias_fold.accumulate = acc_db;
    } else if (db) {
        // two levels: 256 slices of the per-block sums, then the slices
        const int64_t rows = (int64_t)g.N * ptiles;
        const int slices = rows < 256 ? (int)rows : 256;
        const int64_t rps = (rows + slices - 1) / slices;
        float* level1 = bias_part + rows * g.K;
        dim3 g1((unsigned)((g.K + 31) / 32), (unsigned)slices);
        mtl_launch_pdl(ctx, k_colsum, dim3(g1), dim3(256), (size_t)(0), level1, bias_part, rows, g.K, rps, 0);
        MTL_LAUNCHED(ctx);
        mtl_launch_pdl(ctx, k_colsum, dim3((g.K + 31) / 32), dim3(256), (size_t)(0), db, level1, slices, g.K, slices, acc_db);
        MTL_LAUNCHED(ctx);
    }
    const bool x_ready = X_cl && !x3;  // the caller's channels-last copy of X replaces the staging pass
    if (!x_ready) {
        rc = stage_nhwc(ctx, x_hi, x_lo, X, g.N, g.C, g.H * g.W, x3, nullptr);
        if (rc) return rc;
    }
    rc = wgrad_core(ctx, dW, u_hi, u_lo, x_ready ? X_cl : x_hi, x_lo, partial, p, g, acc_dw, x3, bias_fold);
    if (rc) return rc;
    if (ctx->grads_ready_hook) ctx->grads_ready_hook(ctx->grads_ready_user);   // dW and db are enqueued, dX is not
    // input gradient: the same copy of ug is the activation operand; its weights go where X was
    return run_igemm_core(ctx, c, x3, u_hi, u_lo, region, x3 ? region + wt_pad : nullptr);
}
