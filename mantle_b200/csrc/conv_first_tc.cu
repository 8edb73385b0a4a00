// CONV2D + bias + RELU + 2x2 / stride-2 MAXPOOL2D for a network's first layer (few input channels,
// C*R*S <= 32, stride 1, dilation 1) on the tensor cores, plain TF32 mode.
//
// Such a layer has almost no reduction (25 taps for a 5x5 kernel on one channel), so on CUDA cores it
// is bound by issuing FMAs and on the tensor cores by draining the accumulator.  The kernel is built
// around the drain:
//   * GEMM orientation: channels on M, pixels on N, taps on K.  One accumulator column serves TWO
//     pixels: the reduction is doubled to K = 64, k-block 0 holding the patches of pixel set 0 and
//     k-block 1 those of pixel set 1, and the weight tile is [W | 0] in rows 0-63 and [0 | W] in rows
//     64-127.  All 128 TMEM lanes then carry useful rows (64 channels x 2 pixel sets), so all four
//     lane quadrants drain in parallel.
//   * A tile is eight "row pairs" (two adjacent output rows of one image = one pooled row): four per
//     pixel set, 2*OW accumulator columns each.  A TMA box per row pair brings the zero-padded input
//     rows into shared memory; four builder warps expand them into the K-major, 128-byte-swizzled
//     patch tile the tensor core reads (one 128-byte row of 32 taps per pixel); one thread issues
//     the eight MMAs; sixteen epilogue warps (four per lane quadrant, one row pair each) pool in
//     registers and write the pooled values, the argmax indices and the channels-last twin.  So many
//     warps because the pooling is a chain of dependent compares: it needs warps, not width, to
//     fill the issue slots.
//   * The activation never reaches memory; the step is bound by writing the pooled outputs.
// MAXPOOL2D.forward order: window scanned row-major with a strict '>', first maximum wins
// (pool.mojo:44-100 in the reference).
#include <stdlib.h>

#include "common.cuh"
#include "conv.cuh"
#include "sm100.cuh"

namespace {

using namespace sm100;

constexpr int kEpiWarps = 16, kBuildWarps = 4;
constexpr int kThreadsF = (kEpiWarps + kBuildWarps + 2) * 32;  // + TMA producer warp + MMA warp
constexpr int kBuildThreads = kBuildWarps * 32;
constexpr int kPairsPerSet = 4, kPairsPerTile = 2 * kPairsPerSet;
constexpr int kABytes = 2 * 128 * 128;        // two k-blocks of 128 rows x 32 floats
constexpr int kBBlockBytes = 256 * 128;       // one k-block of up to 256 pixel rows
constexpr int kBStageBytes = 2 * kBBlockBytes;
constexpr int kInStages = 2;
constexpr uint64_t kWaitNs = 2000000000ull;

struct FirstParams {
    int N, K, OH, ph, pw;
    int xw, xoff, xstart;      // input box: row stride in floats, column of tap 0 of pixel 0, first x coordinate
    int box_slot;              // floats between the boxes of a stage (multiple of 32)
    int total_pairs;           // N * OH / 2
    int tiles;
    int relu;
    float* pooled;
    int32_t* idx;
    float* pooled_cl;
    const float* Wt;
    const float* bias;
    int* status;
};

template <int R, int S, int C, int OW>
struct FirstCfg {
    static constexpr int CRS = C * R * S;
    static_assert(CRS <= 32, "the taps of one pixel must fit one 128-byte row");
    static_assert(OW % 2 == 0 && 2 * OW <= 64, "a row pair must fit two 32-column TMEM loads");
    static constexpr int IRB = 2 + R - 1;                       // input rows behind a row pair
    static constexpr int XW_MAX = (OW + S - 1 + 3 + 3) / 4 * 4;  // widest box row
    static constexpr int BOX_SLOT = (C * IRB * XW_MAX + 31) / 32 * 32;
    static constexpr int IN_STAGE_BYTES = kPairsPerTile * BOX_SLOT * 4;
    static constexpr int NPX = kPairsPerSet * 2 * OW;            // pixels (accumulator columns) per set
    static constexpr int N_MMA = (NPX + 15) / 16 * 16;
    static_assert(N_MMA <= 256, "accumulator width");
    static constexpr int POW = OW / 2;
    static_assert(POW >= 8 && POW <= 16, "pooled row width");
    // staging row stride: 16-byte aligned rows whose float4 stores spread over all banks
    static constexpr int PST = 20;
    static constexpr int EPI_WARP_BYTES = 32 * PST * 4;
    static constexpr int FIXED_BYTES = 1024 + kABytes + kInStages * IN_STAGE_BYTES + kEpiWarps * EPI_WARP_BYTES + 256;
    // two patch-tile stages when they fit, else one (the builders then wait for the tile's MMAs)
    static constexpr int B_STAGES = FIXED_BYTES + 2 * kBStageBytes <= 232448 ? 2 : 1;
    static constexpr int SMEM_BYTES = FIXED_BYTES + B_STAGES * kBStageBytes;
    static_assert(SMEM_BYTES <= 232448, "shared memory");
};

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Byte offset of element (row, k) of a K-major tile with the 128-byte swizzle: rows of 128 bytes,
// eight-row groups 1024 bytes apart, the 16-byte chunk index XORed with the row inside its group.
__device__ __forceinline__ uint32_t swz_off(int row, int k) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((((k >> 2) ^ (row & 7)) & 7) << 4) + (k & 3) * 4);
}

// 2x2 / stride-2 max pooling of NW windows of one channel: ra holds 2*NW columns of the upper output
// row, rb the same columns of the lower row.  Bias first (so that ties are ties of the stored
// values), then the first maximum in row-major window order, then RELU: when no value of the
// window is positive every activated value is 0 and the first position wins.
template <int NW>
__device__ __forceinline__ void pool_windows(const uint32_t (&ra)[16], const uint32_t (&rb)[16], float bv, int relu,
                                             int ibase, int OW, float (&m)[8], int (&at)[8]) {
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        if (w < NW) {
            const float a = __uint_as_float(ra[2 * w]) + bv, b = __uint_as_float(ra[2 * w + 1]) + bv;
            const float c = __uint_as_float(rb[2 * w]) + bv, d = __uint_as_float(rb[2 * w + 1]) + bv;
            const float m01 = b > a ? b : a, m23 = d > c ? d : c;
            const int i01 = b > a ? 1 : 0, i23 = d > c ? OW + 1 : OW;
            float mm = m23 > m01 ? m23 : m01;
            int ii = m23 > m01 ? i23 : i01;
            if (relu && !(mm > 0.0f)) { mm = 0.0f; ii = 0; }
            m[w] = mm;
            at[w] = ibase + 2 * w + ii;
        } else {
            m[w] = 0.0f;
            at[w] = 0;
        }
    }
}

template <int R, int S, int C, int OW>
__global__ void __launch_bounds__(kThreadsF, 1)
k_conv_first_pool_tc(const __grid_constant__ CUtensorMap mapX, FirstParams p) {
    using Cfg = FirstCfg<R, S, C, OW>;
    constexpr int CRS = Cfg::CRS, IRB = Cfg::IRB, NPX = Cfg::NPX, POW = Cfg::POW, PST = Cfg::PST;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_tile = smem;
    uint8_t* b_tiles = smem + kABytes;
    float* in_tiles = reinterpret_cast<float*>(b_tiles + Cfg::B_STAGES * kBStageBytes);
    uint8_t* epi = reinterpret_cast<uint8_t*>(in_tiles) + kInStages * Cfg::IN_STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(epi + kEpiWarps * Cfg::EPI_WARP_BYTES);
    uint64_t* in_full = bars;            // [kInStages]
    uint64_t* in_empty = bars + 2;       // [kInStages]
    uint64_t* b_full = bars + 4;         // [2]
    uint64_t* b_empty = bars + 6;        // [2]
    uint64_t* acc_full = bars + 8;       // [2]
    uint64_t* acc_empty = bars + 10;     // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kg = blockIdx.y;           // group of 64 output channels
    const int POH = p.OH >> 1;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kInStages; ++s) { mbar_init(&in_full[s], 1); mbar_init(&in_empty[s], kBuildThreads); }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&b_full[s], kBuildThreads); mbar_init(&b_empty[s], 1);
            mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], kEpiWarps);
        }
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&mapX);
    }
    if (warp == kEpiWarps + kBuildWarps + 1) {
        tmem_alloc(tmem_slot, 512);
        tmem_relinquish();
    }
    mtl_pdl_sync();   // the weights read below come from the previous step's optimizer kernel
    // weight tile: k-block b holds W in the rows of pixel set b and zeros in the other 64 rows
    for (int i = threadIdx.x; i < 2 * 128 * 32; i += kThreadsF) {
        const int kb = i >> 12, row = (i >> 5) & 127, k = i & 31;
        const int ch = kg * 64 + (row & 63);
        float v = 0.0f;
        if ((row >> 6) == kb && ch < p.K && k < CRS) v = __ldg(p.Wt + (int64_t)ch * CRS + k);
        *reinterpret_cast<float*>(a_tile + kb * 16384 + swz_off(row, k)) = v;
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == kEpiWarps + kBuildWarps) {
        // ---------------------------------------------------------------- TMA producer: one lane per box
        if (lane < kPairsPerTile) {
            bool ok = true;
            int local = 0;
            for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++local) {
                const int st = local % kInStages;
                const uint32_t ph = (uint32_t)(local / kInStages) & 1u;
                if (!mbar_wait(&in_empty[st], ph ^ 1u, abort_flag, kWaitNs)) ok = false;
                if (__any_sync(0xffu, !ok)) { ok = false; break; }
                if (lane == 0) mbar_arrive_expect_tx(&in_full[st], (uint32_t)(kPairsPerTile * C * IRB * p.xw * 4));
                __syncwarp(0xffu);
                const int g = t * kPairsPerTile + lane;
                const int n = g / POH, pr = g - n * POH;   // n >= N reads zeros (out-of-range box)
                float* dst = in_tiles + st * (Cfg::IN_STAGE_BYTES / 4) + lane * p.box_slot;
                tma_load_4d(dst, &mapX, &in_full[st], p.xstart, 2 * pr - p.ph, 0, n);
            }
            if (!ok && lane == 0) atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else if (warp == kEpiWarps + kBuildWarps + 1) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc = make_idesc_tf32(Cfg::N_MMA, false, false);
            const uint32_t sa = smem_u32(a_tile);
            bool ok = true;
            int local = 0;
            for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++local) {
                const int s = local & 1;
                const uint32_t ph = (uint32_t)(local >> 1) & 1u;
                const int bs = local % Cfg::B_STAGES;
                const uint32_t bph = (uint32_t)(local / Cfg::B_STAGES) & 1u;
                if (!mbar_wait(&acc_empty[s], ph ^ 1u, abort_flag, kWaitNs)) { ok = false; break; }
                if (!mbar_wait(&b_full[bs], bph, abort_flag, kWaitNs)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t sb = smem_u32(b_tiles + bs * kBStageBytes);
                const uint32_t tmem_d = tmem_base + (uint32_t)(s * 256);
#pragma unroll
                for (int kb = 0; kb < 2; ++kb)
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        mma_tf32(tmem_d, desc_k_major(sa + kb * 16384, kk), desc_k_major(sb + kb * kBBlockBytes, kk),
                                 idesc, (kb | kk) ? 1u : 0u);
                mma_commit(&b_empty[bs]);
                mma_commit(&acc_full[s]);
            }
            if (!ok) atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else if (warp >= kEpiWarps) {
        // ---------------------------------------------------------------- patch builders
        const int tb = threadIdx.x - kEpiWarps * 32;
        bool ok = true;
        int local = 0;
        for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++local) {
            const int st = local % kInStages;
            const uint32_t iph = (uint32_t)(local / kInStages) & 1u;
            const int s = local % Cfg::B_STAGES;
            const uint32_t bph = (uint32_t)(local / Cfg::B_STAGES) & 1u;
            if (!mbar_wait(&in_full[st], iph, abort_flag, kWaitNs)) { ok = false; break; }
            if (!mbar_wait(&b_empty[s], bph ^ 1u, abort_flag, kWaitNs)) { ok = false; break; }
            const float* in_st = in_tiles + st * (Cfg::IN_STAGE_BYTES / 4);
            uint8_t* b_st = b_tiles + s * kBStageBytes;
            for (int item = tb; item < 2 * NPX; item += kBuildThreads) {
                const int set = item / NPX, col = item - set * NPX;
                const int rp = col / (2 * OW), rem = col - rp * 2 * OW;
                const int h = rem / OW, ow = rem - h * OW;
                const float* xb = in_st + (set * kPairsPerSet + rp) * p.box_slot + h * p.xw + ow + p.xoff;
                float v[32];
#pragma unroll
                for (int c = 0; c < C; ++c)
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int s2 = 0; s2 < S; ++s2) v[(c * R + r) * S + s2] = xb[(c * IRB + r) * p.xw + s2];
#pragma unroll
                for (int k = CRS; k < 32; ++k) v[k] = 0.0f;
                uint8_t* rowp = b_st + set * kBBlockBytes + (col >> 3) * 1024 + (col & 7) * 128;
#pragma unroll
                for (int ch = 0; ch < 8; ++ch)
                    *reinterpret_cast<float4*>(rowp + ((ch ^ (col & 7)) << 4)) =
                        make_float4(v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]);
            }
            fence_proxy_async_smem();
            mbar_arrive(&b_full[s]);
            mbar_arrive(&in_empty[st]);
        }
        if (!ok && lane == 0) atomicExch(p.status, MTL_ERR_TIMEOUT);
    } else {
        // ---------------------------------------------------------------- epilogue: pool and store
        // warp = (row pair of the set) * 4 + lane quadrant; one row pair per warp per tile
        const int quad = warp & 3, rp = warp >> 2;
        const int set = quad >> 1;
        const int ch0 = kg * 64 + (quad & 1) * 32;
        const int ch = ch0 + lane;
        const float bv = (p.bias && ch < p.K) ? __ldg(p.bias + ch) : 0.0f;
        float* sv = reinterpret_cast<float*>(epi + warp * Cfg::EPI_WARP_BYTES);
        int32_t* si = reinterpret_cast<int32_t*>(sv);
        bool ok = true;
        int local = 0;
        for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++local) {
            const int s = local & 1;
            const uint32_t ph = (uint32_t)(local >> 1) & 1u;
            if (!mbar_wait(&acc_full[s], ph, abort_flag, kWaitNs)) { ok = false; break; }
            tc_fence_after_sync();
            const int g = t * kPairsPerTile + set * kPairsPerSet + rp;
            const int n = g / POH, pr = g - n * POH;
            const int i0 = 2 * pr * OW;
            const bool live = g < p.total_pairs;
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(s * 256 + rp * 2 * OW);
            float* tw = p.pooled_cl ? p.pooled_cl + (((int64_t)n * POH + pr) * POW) * p.K + ch : nullptr;
            const bool tw_ok = live && tw && ch < p.K;
            int at[16];
            __syncwarp();   // the previous tile's read-out of this warp's staging rows is complete
            {   // pooled columns 0-7: accumulator columns 0-15 of both rows
                uint32_t ra[16], rb[16];
                tmem_ld_32x16(taddr, ra);
                tmem_ld_32x16(taddr + OW, rb);
                tmem_ld_wait();
                float m[8];
                pool_windows<8>(ra, rb, bv, p.relu, i0, OW, m, reinterpret_cast<int(&)[8]>(at[0]));
                if (tw_ok) {
#pragma unroll
                    for (int w = 0; w < 8; ++w) tw[(int64_t)w * p.K] = m[w];
                }
                *reinterpret_cast<float4*>(sv + lane * PST) = make_float4(m[0], m[1], m[2], m[3]);
                *reinterpret_cast<float4*>(sv + lane * PST + 4) = make_float4(m[4], m[5], m[6], m[7]);
            }
            {   // pooled columns 8 and up: accumulator columns 16-31 (those past the row are ignored)
                uint32_t ra[16], rb[16];
                tmem_ld_32x16(taddr + 16, ra);
                tmem_ld_32x16(taddr + OW + 16, rb);
                tmem_ld_wait();
                // every TMEM read of this tile is complete: the MMA warp may overwrite the accumulator
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[s]);
                float m[8];
                pool_windows<POW - 8>(ra, rb, bv, p.relu, i0 + 16, OW, m, reinterpret_cast<int(&)[8]>(at[8]));
                if (tw_ok) {
#pragma unroll
                    for (int w = 0; w < POW - 8; ++w) tw[(int64_t)(8 + w) * p.K] = m[w];
                }
                *reinterpret_cast<float4*>(sv + lane * PST + 8) = make_float4(m[0], m[1], m[2], m[3]);
                *reinterpret_cast<float4*>(sv + lane * PST + 12) = make_float4(m[4], m[5], m[6], m[7]);
            }
            __syncwarp();
            // NCHW: 32 channels x POW pooled columns; consecutive lanes take consecutive column pairs
            const int64_t obase = (((int64_t)n * p.K + ch0) * POH + pr) * POW;
            {
                float2 ov[POW / 2];
#pragma unroll
                for (int i = 0; i < POW / 2; ++i) {
                    const int e = lane + 32 * i, cl = e / (POW / 2), pp = e - cl * (POW / 2);
                    ov[i] = *reinterpret_cast<const float2*>(sv + cl * PST + 2 * pp);
                }
                if (live) {
#pragma unroll
                    for (int i = 0; i < POW / 2; ++i) {
                        const int e = lane + 32 * i, cl = e / (POW / 2), pp = e - cl * (POW / 2);
                        if (ch0 + cl < p.K)
                            *reinterpret_cast<float2*>(p.pooled + obase + (int64_t)cl * POH * POW + 2 * pp) = ov[i];
                    }
                }
            }
            if (p.idx) {
                __syncwarp();
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    *reinterpret_cast<int4*>(si + lane * PST + 4 * q4) = make_int4(at[4 * q4], at[4 * q4 + 1], at[4 * q4 + 2], at[4 * q4 + 3]);
                __syncwarp();
                int2 oi[POW / 2];
#pragma unroll
                for (int i = 0; i < POW / 2; ++i) {
                    const int e = lane + 32 * i, cl = e / (POW / 2), pp = e - cl * (POW / 2);
                    oi[i] = *reinterpret_cast<const int2*>(si + cl * PST + 2 * pp);
                }
                if (live) {
#pragma unroll
                    for (int i = 0; i < POW / 2; ++i) {
                        const int e = lane + 32 * i, cl = e / (POW / 2), pp = e - cl * (POW / 2);
                        if (ch0 + cl < p.K)
                            *reinterpret_cast<int2*>(p.idx + obase + (int64_t)cl * POH * POW + 2 * pp) = oi[i];
                    }
                }
            }
        }
        if (!ok && lane == 0) atomicExch(p.status, MTL_ERR_TIMEOUT);
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kEpiWarps + kBuildWarps + 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

template <int R, int S, int C, int OW>
int32_t launch_first(mtl_ctx* ctx, float* pooled, int32_t* idx, float* pooled_cl, const float* X, const float* Wt,
                     const float* bias, const ConvGeom& g, int relu) {
    using Cfg = FirstCfg<R, S, C, OW>;
    FirstParams p;
    p.N = g.N; p.K = g.K; p.OH = g.OH; p.ph = g.ph; p.pw = g.pw;
    const int xs = (g.pw + 3) / 4 * 4;                  // the box starts on a 16-byte boundary left of the padding
    p.xstart = -xs;
    p.xoff = xs - g.pw;
    p.xw = (OW + S - 1 + p.xoff + 3) / 4 * 4;
    p.box_slot = (C * Cfg::IRB * p.xw + 31) / 32 * 32;
    p.total_pairs = g.N * (g.OH / 2);
    p.tiles = (p.total_pairs + kPairsPerTile - 1) / kPairsPerTile;
    p.relu = relu;
    p.pooled = pooled; p.idx = idx; p.pooled_cl = pooled_cl; p.Wt = Wt; p.bias = bias; p.status = ctx->dev_status;
    if (p.xw > Cfg::XW_MAX || p.box_slot > Cfg::BOX_SLOT)
        return mtl_set_error(ctx, MTL_ERR_UNSUPPORTED, "first-layer tensor-core convolution: input box too wide");
    CUtensorMap tm;
    uint64_t dims[4] = {(uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.C, (uint64_t)g.N};
    uint64_t strides[3] = {(uint64_t)g.W * 4, (uint64_t)g.H * g.W * 4, (uint64_t)g.C * g.H * g.W * 4};
    uint32_t box[4] = {(uint32_t)p.xw, (uint32_t)Cfg::IRB, (uint32_t)C, 1u};
    int32_t rc = mtl_encode_tmap(ctx, &tm, X, 4, dims, strides, box, 2);
    if (rc) return rc;
    auto kern = k_conv_first_pool_tc<R, S, C, OW>;
    MTL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    const int kgroups = (g.K + 63) / 64;
    int gx = ctx->sm_count / kgroups;
    if (gx < 1) gx = 1;
    if (gx > p.tiles) gx = p.tiles;
    {
        mtl_prof_scope prof(ctx, MTL_PROF_CONV_FIRST);
        mtl_launch_pdl(ctx, kern, dim3(dim3(gx, kgroups)), dim3(kThreadsF), (size_t)(Cfg::SMEM_BYTES), tm, p);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

// ------------------------------------------------------------------------------------------------
// Kernel and bias gradient of the same layer from the POOLED upper gradient (CONV2D.backward of
// RELU.backward of MAXPOOL2D.backward), plain TF32 mode.
//
// GEMM: D[(set, channel)][(set', tap)] += sum over pixels of dY[(set, channel)][pixel] * patch[(set', tap)][pixel]
// with two pixel sets so that all 128 accumulator rows work (the blocks with set == set' are the
// result, the other two are discarded).  A tile is four output rows of one image: set 0 the upper
// row pair, set 1 the lower one, 2*OW pixels on K.  Builder warps rebuild the dense gradient of a
// row pair in the K-major operand tile (every pooled element writes its whole 2x2 window: the
// gradient where the argmax was, zeros elsewhere, nothing if RELU was inactive) and lay the input
// rows out as shifted copies, one per tap; tap C*R*S is a row of ones, so its column is the bias
// gradient.  The accumulator stays in tensor memory for the whole kernel; each CTA writes one partial
// result, summed by a second launch.
constexpr int kWBuildWarps = 16, kWBuildThreads = kWBuildWarps * 32;
constexpr int kThreadsW = (kWBuildWarps + 2) * 32;
constexpr int kWABytes = 2 * 128 * 128;   // (set, channel) rows, two k-blocks of 32 pixels
constexpr int kWBBytes = 2 * 64 * 128;    // (set', tap) rows
constexpr int kWStageBytes = kWABytes + kWBBytes;

struct FirstWgradParams {
    int N, K, OH, ph, pw;
    int xw, xoff, xstart, box_floats;
    int tiles;                 // N * (OH / 4)
    int relu;
    const float* pg;           // pooled upper gradient [N, K, OH/2, OW/2]
    const int32_t* idx;        // argmax indices of the pooling
    const float* pv;           // pooled output (RELU mask), may be null when relu == 0
    float* part;               // [gridDim.x][K][32]: taps 0 .. C*R*S-1, then the bias column
    int* status;
};

template <int R, int S, int C, int OW>
struct FirstWgradCfg {
    static constexpr int CRS = C * R * S;
    static_assert(CRS <= 31, "one spare tap row carries the bias gradient");
    static_assert(OW % 4 == 0, "four-pixel chunks must not straddle output rows");
    static constexpr int IRB = 4 + R - 1;
    static constexpr int XW_MAX = (OW + S - 1 + 3 + 3) / 4 * 4;
    static constexpr int IN_STAGE_BYTES = (C * IRB * XW_MAX * 4 + 127) / 128 * 128;
    static constexpr int PX = 2 * OW;            // pixels of a row pair = K extent of a set
    static constexpr int KSTEPS = PX / 8;        // MMAs per tile
    static constexpr int POW = OW / 2;
    static constexpr int QPC = 2 * POW / 4;      // float4 loads per channel and tile (both row pairs)
    static constexpr int ITEMS = 64 * QPC;
    static constexpr int IPT = (ITEMS + kWBuildThreads - 1) / kWBuildThreads;
    static constexpr int SMEM_BYTES = 1024 + 2 * kWStageBytes + 2 * IN_STAGE_BYTES + 64 * 33 * 4 + 256;
    static_assert(SMEM_BYTES <= 232448, "shared memory");
};

template <int R, int S, int C, int OW>
__global__ void __launch_bounds__(kThreadsW, 1)
k_conv_first_wgrad_tc(const __grid_constant__ CUtensorMap mapX, FirstWgradParams p) {
    using Cfg = FirstWgradCfg<R, S, C, OW>;
    constexpr int CRS = Cfg::CRS, IRB = Cfg::IRB, PX = Cfg::PX, POW = Cfg::POW, QPC = Cfg::QPC, IPT = Cfg::IPT;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ab = smem;                                                    // 2 stages of {A, B}
    float* in_tiles = reinterpret_cast<float*>(smem + 2 * kWStageBytes);
    float* xch = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(in_tiles) + 2 * Cfg::IN_STAGE_BYTES);  // [64][33]
    uint64_t* bars = reinterpret_cast<uint64_t*>(xch + 64 * 33);
    uint64_t* in_full = bars;        // [2]
    uint64_t* in_empty = bars + 2;   // [2]
    uint64_t* ab_full = bars + 4;    // [2]
    uint64_t* ab_empty = bars + 6;   // [2]
    uint64_t* acc_done = bars + 8;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kg = blockIdx.y;
    const int POH = p.OH >> 1, TPI = POH >> 1;   // tiles per image

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&in_full[s], 1); mbar_init(&in_empty[s], kWBuildThreads);
            mbar_init(&ab_full[s], kWBuildThreads); mbar_init(&ab_empty[s], 1);
        }
        mbar_init(acc_done, 1);
        *abort_flag = 0;
        fence_barrier_init();
        prefetch_tensormap(&mapX);
    }
    if (warp == kWBuildWarps + 1) {
        tmem_alloc(tmem_slot, 64);
        tmem_relinquish();
    }
    // operand tiles start as zeros; the tap row C*R*S of each set is ones (bias gradient)
    for (int i = threadIdx.x; i < 2 * kWStageBytes / 4; i += kThreadsW) reinterpret_cast<float*>(ab)[i] = 0.0f;
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * 2 * 2 * 32; i += kThreadsW) {
        const int st = i >> 7, kb = (i >> 6) & 1, set = (i >> 5) & 1, k = i & 31;
        *reinterpret_cast<float*>(ab + st * kWStageBytes + kWABytes + kb * (64 * 128) + swz_off(set * 32 + CRS, k)) = 1.0f;
    }
    fence_proxy_async_smem();
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    mtl_pdl_sync();   // everything above touched only shared / tensor memory

    if (warp == kWBuildWarps) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            bool ok = true;
            int local = 0;
            for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++local) {
                const int st = local & 1;
                const uint32_t ph = (uint32_t)(local >> 1) & 1u;
                if (!mbar_wait(&in_empty[st], ph ^ 1u, abort_flag, kWaitNs)) { ok = false; break; }
                mbar_arrive_expect_tx(&in_full[st], (uint32_t)(p.box_floats * 4));
                const int n = t / TPI, j = t - n * TPI;
                tma_load_4d(reinterpret_cast<uint8_t*>(in_tiles) + st * Cfg::IN_STAGE_BYTES, &mapX, &in_full[st], p.xstart,
                            4 * j - p.ph, 0, n);
            }
            if (!ok) atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else if (warp == kWBuildWarps + 1) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc = make_idesc_tf32(64, false, false);
            bool ok = true;
            int local = 0;
            for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++local) {
                const int s = local & 1;
                const uint32_t ph = (uint32_t)(local >> 1) & 1u;
                if (!mbar_wait(&ab_full[s], ph, abort_flag, kWaitNs)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t sa = smem_u32(ab + s * kWStageBytes);
                const uint32_t sb = sa + kWABytes;
#pragma unroll
                for (int ks = 0; ks < Cfg::KSTEPS; ++ks) {
                    const int kb = ks >> 2, kk = ks & 3;
                    mma_tf32(tmem_base, desc_k_major(sa + kb * 16384, kk), desc_k_major(sb + kb * (64 * 128), kk), idesc,
                             (local | ks) ? 1u : 0u);
                }
                mma_commit(&ab_empty[s]);
            }
            if (ok) mma_commit(acc_done);
            else atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else {
        // ---------------------------------------------------------------- operand builders
        const int tb = threadIdx.x;
        // Everything that does not depend on the tile is worked out once: where this thread's pooled
        // elements land in the gradient tile (upper and lower row of their windows), and which
        // four-pixel pieces of which tap rows it copies.  Odd lanes take the elements of a quad in the
        // order 1, 0, 3, 2: with every lane on the same element parity the 8-byte stores of a warp
        // would use only half of the banks.
        const int swap = lane & 1;
        uint32_t a_up[IPT][4], a_lo[IPT][4];
        int a_i0[IPT][4];
        int a_src[IPT];     // element offset of the quad inside its tile's data, -1: nothing to do
#pragma unroll
        for (int i = 0; i < IPT; ++i) {
            const int it = tb + i * kWBuildThreads;
            const int cl = it / QPC, q = it - cl * QPC;
            a_src[i] = (it < Cfg::ITEMS && kg * 64 + cl < p.K) ? ((kg * 64 + cl) * POH * POW + 4 * q) : -1;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int e = 4 * q + (u ^ swap);
                const int set = e / POW, pw = e - set * POW;
                const int row = set * 64 + (cl & 63);
                const int j0 = 2 * pw, j1 = OW + 2 * pw;
                a_up[i][u] = (uint32_t)((j0 >> 5) * 16384) + swz_off(row, j0 & 31);
                a_lo[i][u] = (uint32_t)((j1 >> 5) * 16384) + swz_off(row, j1 & 31);
                a_i0[i][u] = 2 * set * OW + 2 * pw;
            }
        }
        constexpr int B_ITEMS = 2 * CRS * (PX / 4), BPT = (B_ITEMS + kWBuildThreads - 1) / kWBuildThreads;
        int b_src[BPT];
        uint32_t b_dst[BPT];
#pragma unroll
        for (int i = 0; i < BPT; ++i) {
            const int it = tb + i * kWBuildThreads;
            const int c4 = it % (PX / 4), rest = it / (PX / 4);
            const int tap = rest % CRS, set = (rest / CRS) & 1;
            const int cc = tap / (R * S), r = (tap / S) % R, s2 = tap % S;
            const int px = 4 * c4, h = px / OW, ow = px - h * OW;
            b_src[i] = it < B_ITEMS ? (cc * IRB + 2 * set + h + r) * p.xw + ow + s2 + p.xoff : -1;
            b_dst[i] = (uint32_t)((px >> 5) * (64 * 128)) + swz_off(set * 32 + tap, px & 31);
        }
        // Pooled gradient, argmax index and pooled value of this thread's elements, for two tiles: the
        // loads of a register set are issued as soon as the set's tile has been consumed, i.e. two
        // tiles ahead of their use (one tile of MMAs is shorter than a DRAM round trip).
        float4 gA[IPT], vA[IPT], gB[IPT], vB[IPT];
        int4 iA[IPT], iB[IPT];
        auto fetch = [&](int t, float4 (&g)[IPT], int4 (&ix)[IPT], float4 (&pvr)[IPT]) {
            if (t >= p.tiles) return;
            const int n = t / TPI, j = t - n * TPI;
            const int tile_off = n * p.K * POH * POW + 2 * j * POW;   // below 2^31: checked by the host
#pragma unroll
            for (int i = 0; i < IPT; ++i) {
                if (a_src[i] >= 0) {
                    const int o = tile_off + a_src[i];
                    g[i] = __ldg(reinterpret_cast<const float4*>(p.pg + o));
                    ix[i] = __ldg(reinterpret_cast<const int4*>(p.idx + o));
                    if (p.relu) pvr[i] = __ldg(reinterpret_cast<const float4*>(p.pv + o));
                }
            }
        };
        bool ok = true;
        auto build = [&](int t, int local, float4 (&g)[IPT], int4 (&ix)[IPT], float4 (&pvr)[IPT]) {
            const int st = local & 1;
            const uint32_t ph = (uint32_t)(local >> 1) & 1u;
            const int j = t % TPI;
            if (!mbar_wait(&ab_empty[st], ph ^ 1u, abort_flag, kWaitNs)) { ok = false; return; }
            uint8_t* a_st = ab + st * kWStageBytes;
            uint8_t* b_st = a_st + kWABytes;
            // dense gradient rows from the pooled elements in registers
            const int tile_i0 = 4 * j * OW;
#pragma unroll
            for (int i = 0; i < IPT; ++i) {
                if (a_src[i] >= 0) {
                    const float gv[4] = {swap ? g[i].y : g[i].x, swap ? g[i].x : g[i].y, swap ? g[i].w : g[i].z, swap ? g[i].z : g[i].w};
                    const float pvv[4] = {swap ? pvr[i].y : pvr[i].x, swap ? pvr[i].x : pvr[i].y, swap ? pvr[i].w : pvr[i].z,
                                          swap ? pvr[i].z : pvr[i].w};
                    const int iv[4] = {swap ? ix[i].y : ix[i].x, swap ? ix[i].x : ix[i].y, swap ? ix[i].w : ix[i].z, swap ? ix[i].z : ix[i].w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const float val = (!p.relu || pvv[u] > 0.0f) ? gv[u] : 0.0f;   // RELU.backward: x > 0 ? ug : 0
                        const int c = iv[u] - tile_i0 - a_i0[i][u];                    // 0, 1, OW, OW + 1
                        const bool lower = c >= OW;
                        const bool right = (c & 1) != 0;                               // OW is even
                        const float2 hit = right ? make_float2(0.0f, val) : make_float2(val, 0.0f);
                        const float2 zero = make_float2(0.0f, 0.0f);
                        *reinterpret_cast<float2*>(a_st + a_up[i][u]) = lower ? zero : hit;
                        *reinterpret_cast<float2*>(a_st + a_lo[i][u]) = lower ? hit : zero;
                    }
                }
            }
            fetch(t + 2 * (int)gridDim.x, g, ix, pvr);
            // input rows as shifted copies: row (set', tap), four pixels per store
            if (!mbar_wait(&in_full[st], ph, abort_flag, kWaitNs)) { ok = false; return; }
            const float* xin = in_tiles + st * (Cfg::IN_STAGE_BYTES / 4);
#pragma unroll
            for (int i = 0; i < BPT; ++i) {
                if (b_src[i] >= 0) {
                    const float* src = xin + b_src[i];
                    *reinterpret_cast<float4*>(b_st + b_dst[i]) = make_float4(src[0], src[1], src[2], src[3]);
                }
            }
            fence_proxy_async_smem();
            mbar_arrive(&ab_full[st]);
            mbar_arrive(&in_empty[st]);
        };
#pragma unroll
        for (int i = 0; i < IPT; ++i) {
            gA[i] = gB[i] = vA[i] = vB[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            iA[i] = iB[i] = make_int4(0, 0, 0, 0);
        }
        fetch(blockIdx.x, gA, iA, vA);
        fetch(blockIdx.x + gridDim.x, gB, iB, vB);
        for (int t = blockIdx.x, local = 0; t < p.tiles && ok; t += 2 * gridDim.x, local += 2) {
            build(t, local, gA, iA, vA);
            if (!ok || t + (int)gridDim.x >= p.tiles) break;
            build(t + gridDim.x, local + 1, gB, iB, vB);
        }
        if (!ok && lane == 0) atomicExch(p.status, MTL_ERR_TIMEOUT);

        // ------------------------------------------------------------ the CTA's partial result
        if (warp < 4) {
            const int quad = warp, set = quad >> 1, cl = (quad & 1) * 32 + lane;
            uint32_t v[32];
            bool done = ok && mbar_wait(acc_done, 0u, abort_flag, kWaitNs);
            if (!done && lane == 0) atomicExch(p.status, MTL_ERR_TIMEOUT);
            tc_fence_after_sync();
            tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(set * 32), v);
            tmem_ld_wait();
            if (set == 1) {
#pragma unroll
                for (int k = 0; k < 32; ++k) xch[cl * 33 + k] = __uint_as_float(v[k]);
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int ch = kg * 64 + cl;
            if (set == 0 && ch < p.K && done) {
                float4* dst = reinterpret_cast<float4*>(p.part + ((int64_t)blockIdx.x * p.K + ch) * 32);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    dst[k] = make_float4(__uint_as_float(v[4 * k]) + xch[cl * 33 + 4 * k],
                                         __uint_as_float(v[4 * k + 1]) + xch[cl * 33 + 4 * k + 1],
                                         __uint_as_float(v[4 * k + 2]) + xch[cl * 33 + 4 * k + 2],
                                         __uint_as_float(v[4 * k + 3]) + xch[cl * 33 + 4 * k + 3]);
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == kWBuildWarps + 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 64);
    }
}

// Sums the CTAs' partial results in a fixed order: one block per output channel, 32 columns x 8
// slices of the partials, the slices combined through shared memory.  Column C*R*S is the bias gradient.
__global__ void __launch_bounds__(256) k_first_wgrad_reduce(float* __restrict__ dW, float* __restrict__ db,
                                                            const float* __restrict__ part, int K, int CRS, int nparts,
                                                            int acc_dw, int acc_db) {
    mtl_pdl_sync();
    __shared__ float sm[8][33];
    const int ch = blockIdx.x, col = threadIdx.x & 31, slice = threadIdx.x >> 5;
    float s = 0.0f;
    for (int q = slice; q < nparts; q += 8) s += part[((int64_t)q * K + ch) * 32 + col];
    sm[slice][col] = s;
    __syncthreads();
    if (slice == 0) {
        float t = 0.0f;
#pragma unroll
        for (int j = 0; j < 8; ++j) t += sm[j][col];
        if (col < CRS && dW) {
            float* o = dW + (int64_t)ch * CRS + col;
            *o = acc_dw ? *o + t : t;
        } else if (col == CRS && db) {
            db[ch] = acc_db ? db[ch] + t : t;
        }
    }
}

template <int R, int S, int C, int OW>
int32_t launch_first_wgrad(mtl_ctx* ctx, float* dW, float* db, const float* pg, const int32_t* pidx, const float* pv,
                           const float* X, const ConvGeom& g, int relu, int acc_dw, int acc_db) {
    using Cfg = FirstWgradCfg<R, S, C, OW>;
    FirstWgradParams p;
    p.N = g.N; p.K = g.K; p.OH = g.OH; p.ph = g.ph; p.pw = g.pw;
    const int xs = (g.pw + 3) / 4 * 4;
    p.xstart = -xs;
    p.xoff = xs - g.pw;
    p.xw = (OW + S - 1 + p.xoff + 3) / 4 * 4;
    p.box_floats = C * Cfg::IRB * p.xw;
    p.tiles = g.N * (g.OH / 4);
    p.relu = relu;
    p.pg = pg; p.idx = pidx; p.pv = pv; p.status = ctx->dev_status;
    if (p.xw > Cfg::XW_MAX)
        return mtl_set_error(ctx, MTL_ERR_UNSUPPORTED, "first-layer tensor-core gradient: input box too wide");
    const int kgroups = (g.K + 63) / 64;
    int gx = ctx->sm_count / kgroups;
    if (gx < 1) gx = 1;
    if (gx > p.tiles) gx = p.tiles;
    void* ws;
    int32_t rc = mtl_workspace(ctx, (size_t)gx * g.K * 32 * 4, &ws);
    if (rc) return rc;
    p.part = (float*)ws;
    CUtensorMap tm;
    uint64_t dims[4] = {(uint64_t)g.W, (uint64_t)g.H, (uint64_t)g.C, (uint64_t)g.N};
    uint64_t strides[3] = {(uint64_t)g.W * 4, (uint64_t)g.H * g.W * 4, (uint64_t)g.C * g.H * g.W * 4};
    uint32_t box[4] = {(uint32_t)p.xw, (uint32_t)Cfg::IRB, (uint32_t)C, 1u};
    rc = mtl_encode_tmap(ctx, &tm, X, 4, dims, strides, box, 2);
    if (rc) return rc;
    auto kern = k_conv_first_wgrad_tc<R, S, C, OW>;
    MTL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    {
        mtl_prof_scope prof(ctx, MTL_PROF_CONV_FIRST);
        mtl_launch_pdl(ctx, kern, dim3(dim3(gx, kgroups)), dim3(kThreadsW), (size_t)(Cfg::SMEM_BYTES), tm, p);
    }
    MTL_LAUNCHED(ctx);
    mtl_launch_pdl(ctx, k_first_wgrad_reduce, dim3(g.K), dim3(256), (size_t)(0), dW, db, p.part, g.K, Cfg::CRS, gx, acc_dw, acc_db);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

}  // namespace

#define MTL_FIRST_TC_CASES(X_) X_(5, 5, 1, 28) X_(3, 3, 1, 28) X_(5, 5, 1, 32) X_(3, 3, 3, 32)

bool mtl_conv_first_pool_tc_supported(const ConvGeom& g, const float* X, const float* pooled, const int32_t* idx) {
    if (!mtl_global_tuning().conv_first_tc) return false;
    if (g.sh != 1 || g.sw != 1 || g.dh != 1 || g.dw != 1) return false;
    if (g.OH % 2 || g.OW % 2 || g.W % 4) return false;
    if ((reinterpret_cast<uintptr_t>(X) & 15u) || !pooled) return false;
    if ((reinterpret_cast<uintptr_t>(pooled) & 7u) || (reinterpret_cast<uintptr_t>(idx) & 7u)) return false;  // paired stores
    if (g.ph < 0 || g.pw < 0 || g.ph > g.R - 1 || g.pw > g.S - 1) return false;
    if ((int64_t)g.N * g.K * g.OH * g.OW >= (1ll << 31)) return false;
    if ((int64_t)g.N * (g.OH / 2) < 64) return false;   // too few row pairs to fill the tiles
#define X_(R_, S_, C_, OW_) if (g.R == R_ && g.S == S_ && g.C == C_ && g.OW == OW_) return true;
    MTL_FIRST_TC_CASES(X_)
#undef X_
    return false;
}

int32_t mtl_conv_first_pool_tc(mtl_ctx* ctx, float* pooled, int32_t* idx, float* pooled_cl, const float* X,
                               const float* Wt, const float* bias, const ConvGeom& g, int relu) {
#define X_(R_, S_, C_, OW_)                                               \
    if (g.R == R_ && g.S == S_ && g.C == C_ && g.OW == OW_)               \
        return launch_first<R_, S_, C_, OW_>(ctx, pooled, idx, pooled_cl, X, Wt, bias, g, relu);
    MTL_FIRST_TC_CASES(X_)
#undef X_
    return mtl_set_error(ctx, MTL_ERR_UNSUPPORTED, "first-layer tensor-core convolution: geometry not instantiated");
}

bool mtl_conv_first_wgrad_tc_supported(const ConvGeom& g, const float* X, const float* pg, const int32_t* pidx,
                                       const float* pv) {
    if (!mtl_conv_first_pool_tc_supported(g, X, pg, pidx)) return false;
    if (g.OH % 4) return false;   // a tile is two whole row pairs of one image
    if (((reinterpret_cast<uintptr_t>(pg) | reinterpret_cast<uintptr_t>(pidx) | reinterpret_cast<uintptr_t>(pv)) & 15u)) return false;
    if (((g.OH / 2) * (g.OW / 2)) % 4) return false;   // 16-byte loads from every channel plane
    return true;
}

int32_t mtl_conv_first_wgrad_tc(mtl_ctx* ctx, float* dW, float* db, const float* pg, const int32_t* pidx,
                                const float* pv, const float* X, const ConvGeom& g, int relu, int acc_dw, int acc_db) {
#define X_(R_, S_, C_, OW_)                                               \
    if (g.R == R_ && g.S == S_ && g.C == C_ && g.OW == OW_)               \
        return launch_first_wgrad<R_, S_, C_, OW_>(ctx, dW, db, pg, pidx, pv, X, g, relu, acc_dw, acc_db);
    MTL_FIRST_TC_CASES(X_)
#undef X_
    return mtl_set_error(ctx, MTL_ERR_UNSUPPORTED, "first-layer tensor-core gradient: geometry not instantiated");
}
