// OP.DOT on the 5th-generation tensor cores: C[M,N] (+)= op(A) . op(B) with tcgen05.mma
// kind::tf32, fp32 accumulators in tensor memory, operands staged by TMA into 128-byte-swizzled
// shared memory.  One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer (one lane), ring of STAGES operand buffers
//   warp 1      MMA issuer (one lane); owns the tensor-memory allocation
//   warps 2-5   epilogue: tcgen05.ld -> registers -> global, overlapped with the next tile's
//               main loop through two accumulator buffers in tensor memory
// The same kernel serves the three products of DOT: forward (A row-major = K-major,
// B row-major = N-major), dA = ug . B^T (both K-major) and dB = A^T . ug (both MN-major); no
// transpose pass is needed (the reference transposes physically, matmul.mojo:175-210).
// 3xTF32: the operands are split beforehand into tf32-exact hi and residual lo arrays and the K
// loop runs over the three products lo*hi, hi*lo, hi*hi into the same accumulator.
#include "common.cuh"
#include "sm100.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128;
constexpr int BK = 32;  // 32 fp32 = one 128-byte swizzle row
constexpr int kThreads = 192;
constexpr uint64_t kWaitBudgetNs = 4000000000ull;  // 4 s: far beyond any legitimate wait

// MT = 2: a CTA owns 256 rows, i.e. two M = 128 instructions per k step that share the B tile.  That
// halves the operand rows fetched per flop (the TMA unit, not the tensor pipe, limits the 128-row
// tile) at the price of the second accumulator buffer: the epilogue no longer overlaps the next
// tile's main loop, which only matters for short K.
template <int BN, int MT>
struct Cfg {
    static constexpr int kStages = MT == 2 ? 3 : (BN == 256 ? 4 : 6);
    static constexpr int kABytes = MT * BM * BK * 4;
    static constexpr int kBBytes = BN * BK * 4;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kAccs = MT == 2 ? 1 : 2;        // accumulator sets in tensor memory
    static constexpr int kTmemCols = 2 * BN;             // 2 sets x BN, or 1 set x 2 halves x BN
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

struct GemmParams {
    int M, N, K;
    int nseg;           // 1 (plain tf32) or 3 (hi/lo split products)
    int segA[3], segB[3];  // which map (0 = hi, 1 = lo) each K segment reads
    float* C;
    int accumulate;
    int32_t* status;
    int a3d, b3d;     // MN-major operand fetched as one 3-D box {32, BK, chunks} instead of one box per chunk
    int stages;       // ring depth actually used (<= the configuration's maximum)
    // Stream-K schedule (sk != 0): the tiles' k-blocks, laid end to end, are dealt out evenly over the
    // CTAs, so that a problem with fewer tiles than SMs -- or a tile count that leaves most of the last
    // wave idle -- still keeps every SM busy.  A CTA then works on up to two partial tiles (the first and
    // the last of its range).  Every part of a split tile is written to scratch memory; the CTA that
    // finishes the last part of a tile (a ticket counter per tile) adds the parts in ascending k order
    // and stores the tile, so the result does not depend on which CTA runs when.
    int sk;
    int sk_grid;            // CTAs of the launch: at most four per tile, so that a tile has few parts
    long long sk_q, sk_r;   // CTA c covers units [c*q + min(c, r), (c+1)*q + min(c+1, r))
    float* sk_scratch;      // [gridDim.x][2][tile rows][BN]
    int32_t* sk_tickets;    // one counter per tile, zero between launches
};

// Walks the (tile, k-block range) segments of one CTA; identical in the three roles of the kernel.
struct SegIter {
    int sk, G, num_tiles, kb_total, t, first;
    long long u, u_end;
    __device__ __forceinline__ static long long start_of(long long c, long long q, long long r) { return c * q + (c < r ? c : r); }
    __device__ __forceinline__ void init(const GemmParams& p, int num_tiles_, int kb_total_) {
        sk = p.sk; G = gridDim.x; num_tiles = num_tiles_; kb_total = kb_total_; t = blockIdx.x; first = 1;
        u = start_of(blockIdx.x, p.sk_q, p.sk_r);
        u_end = start_of(blockIdx.x + 1, p.sk_q, p.sk_r);
    }
    // slot: -1 for a whole tile, else which of this CTA's two scratch tiles the part goes to
    __device__ __forceinline__ bool next(int& tile, int& kb0, int& kb1, int& slot) {
        if (!sk) {
            if (t >= num_tiles) return false;
            tile = t; kb0 = 0; kb1 = kb_total; slot = -1; t += G;
            return true;
        }
        if (u >= u_end) return false;
        tile = (int)(u / kb_total);
        kb0 = (int)(u - (long long)tile * kb_total);
        const long long left = u_end - u;
        kb1 = (long long)kb0 + left < (long long)kb_total ? kb0 + (int)left : kb_total;
        slot = (kb0 == 0 && kb1 == kb_total) ? -1 : (first ? 0 : 1);
        first = 0;
        u += kb1 - kb0;
        return true;
    }
};

// The CTA whose range contains unit u (inverse of SegIter::start_of).
__device__ __forceinline__ int cta_of_unit(long long u, long long q, long long r) {
    return u < (q + 1) * r ? (int)(u / (q + 1)) : (int)(r + (u - (q + 1) * r) / q);
}

// Tile order: groups of 16 tile-rows; inside a group the tile-column changes slowest so that
// CTAs running at the same time share B tiles and a bounded set of A tiles in L2.
__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
    constexpr int G = 16;
    int per_group = G * tiles_n;
    int g = t / per_group;
    int r = t - g * per_group;
    int rows = min(G, tiles_m - g * G);
    tm = g * G + r % rows;
    tn = r / rows;
}

template <int BN, bool A_MN, bool B_MN, int MT>
__global__ void __launch_bounds__(kThreads, 1)
k_gemm_tf32(const __grid_constant__ CUtensorMap mapA0, const __grid_constant__ CUtensorMap mapA1,
            const __grid_constant__ CUtensorMap mapB0, const __grid_constant__ CUtensorMap mapB1, GemmParams p) {
    using C = Cfg<BN, MT>;
    constexpr int BMT = BM * MT;  // rows of a CTA tile
    extern __shared__ uint8_t smem_raw[];
    // 128-byte swizzle needs 1024-byte aligned tiles
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* tiles = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStageBytes);
    uint64_t* full = bars;                       // [kStages]
    uint64_t* empty = bars + C::kStages;         // [kStages]
    uint64_t* tmem_full = bars + 2 * C::kStages;  // [2]
    uint64_t* tmem_empty = tmem_full + 2;         // [2]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* fold_flag = abort_flag + 1;   // epilogue warps: does this CTA fold the tile it just finished a part of

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int tiles_m = (p.M + BMT - 1) / BMT;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int kb_per_seg = (p.K + BK - 1) / BK;
    const int kb_total = kb_per_seg * p.nseg;

    if (threadIdx.x == 0) {
        for (int s = 0; s < p.stages; ++s) {
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

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer ----------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            SegIter it;
            it.init(p, num_tiles, kb_total);
            int t, kb0, kb1, slot;
            while (ok && it.next(t, kb0, kb1, slot)) {
                int tm, tn;
                tile_coords(t, tiles_m, tiles_n, tm, tn);
                const int m0 = tm * BMT, n0 = tn * BN;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&empty[stage], phase ^ 1u, abort_flag, kWaitBudgetNs)) { ok = false; break; }
                    const int seg = kb / kb_per_seg;
                    const int k0 = (kb - seg * kb_per_seg) * BK;
                    const CUtensorMap* ma = p.segA[seg] ? &mapA1 : &mapA0;
                    const CUtensorMap* mb = p.segB[seg] ? &mapB1 : &mapB0;
                    uint8_t* sa = tiles + stage * C::kStageBytes;
                    uint8_t* sb = sa + C::kABytes;
                    mbar_arrive_expect_tx(&full[stage], C::kStageBytes);
                    if (A_MN) {
                        // A stored [K, M]: chunks of 32 m x 32 k, 4 KB each
                        if (p.a3d) {
                            tma_load_3d(sa, ma, &full[stage], 0, k0, m0 / 32);
                        } else {
#pragma unroll
                            for (int c = 0; c < BMT / 32; ++c)
                                tma_load_2d(sa + c * 4096, ma, &full[stage], m0 + c * 32, k0);
                        }
                    } else {
                        tma_load_2d(sa, ma, &full[stage], k0, m0);
                    }
                    if (B_MN) {
                        if (p.b3d) {
                            tma_load_3d(sb, mb, &full[stage], 0, k0, n0 / 32);
                        } else {
#pragma unroll
                            for (int c = 0; c < BN / 32; ++c)
                                tma_load_2d(sb + c * 4096, mb, &full[stage], n0 + c * 32, k0);
                        }
                    } else {
                        tma_load_2d(sb, mb, &full[stage], k0, n0);
                    }
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------- MMA issuer ------------
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc_tf32(BN, A_MN, B_MN);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int local = 0;
            SegIter it;
            it.init(p, num_tiles, kb_total);
            int t, kb0, kb1, slot;
            for (; ok && it.next(t, kb0, kb1, slot); ++local) {
                const int acc = local % C::kAccs;
                const uint32_t acc_phase = (uint32_t)(local / C::kAccs) & 1u;
                if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, abort_flag, kWaitBudgetNs)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(&full[stage], phase, abort_flag, kWaitBudgetNs)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(tiles + stage * C::kStageBytes);
                    const uint32_t sb = sa + C::kABytes;
#pragma unroll
                    for (int kk = 0; kk < BK / 8; ++kk) {
                        const uint64_t db = B_MN ? desc_mn_major(sb, kk) : desc_k_major(sb, kk);
#pragma unroll
                        for (int h = 0; h < MT; ++h) {  // the halves of a 256-row tile: 16 KB apart in both layouts
                            const uint32_t sah = sa + (uint32_t)h * (BM * BK * 4);
                            const uint64_t da = A_MN ? desc_mn_major(sah, kk) : desc_k_major(sah, kk);
                            mma_tf32(tmem_d + (uint32_t)(h * BN), da, db, idesc, (kb > kb0 || kk) ? 1u : 0u);
                        }
                    }
                    mma_commit(&empty[stage]);  // frees the stage once these MMAs have read it
                    if (++stage == p.stages) { stage = 0; phase ^= 1u; }
                }
                if (ok) mma_commit(&tmem_full[acc]);
            }
            if (!ok) atomicExch(p.status, MTL_ERR_TIMEOUT);
        }
    } else {
        // ------------------------------------------------------------- epilogue --------------
        const int quad = warp & 3;  // tensor-memory lanes [32*quad, 32*quad + 32)
        const bool vec_ok = (p.N % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.C) & 15u) == 0);
        bool ok = true;
        int local = 0;
        SegIter it;
        it.init(p, num_tiles, kb_total);
        int t, kb0, kb1, slot;
        for (; ok && it.next(t, kb0, kb1, slot); ++local) {
            int tm, tn;
            tile_coords(t, tiles_m, tiles_n, tm, tn);
            const int acc = local % C::kAccs;
            const uint32_t acc_phase = (uint32_t)(local / C::kAccs) & 1u;
            if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, kWaitBudgetNs)) { ok = false; break; }
            tc_fence_after_sync();
            const int n_base = tn * BN;
            if (slot >= 0) {
                // ---- a part of a split tile: park it in scratch memory, then see who finishes the tile
                float* part = p.sk_scratch + ((size_t)blockIdx.x * 2 + slot) * ((size_t)BMT * BN);
#pragma unroll 1
                for (int hc = 0; hc < MT * (BN / 32); ++hc) {
                    const int h = hc / (BN / 32), c = hc - h * (BN / 32);
                    const int row = h * BM + quad * 32 + lane;
                    uint32_t r[32];
                    tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)((acc + h) * BN + c * 32), r);
                    tmem_ld_wait();
                    // layout of a part: [chunk of 32 columns][group of 4 columns][row of the 128-row half]: the
                    // 32 lanes of a warp write 512 contiguous bytes per store
                    float4* dst = reinterpret_cast<float4*>(part) + (size_t)hc * 8 * 128 + quad * 32 + lane;
                    (void)row;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        dst[j * 128] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                   __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                }
                tc_fence_before_sync();
                mbar_arrive(&tmem_empty[acc]);          // the accumulator is free for the next segment
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const long long u_lo = (long long)t * kb_total, u_hi = u_lo + kb_total - 1;
                const int c_lo = cta_of_unit(u_lo, p.sk_q, p.sk_r), c_hi = cta_of_unit(u_hi, p.sk_q, p.sk_r);
                if (threadIdx.x == 64) *fold_flag = atomicAdd(&p.sk_tickets[t], 1) == c_hi - c_lo;
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (!*fold_flag) continue;
                __threadfence();
                // ---- the last part is in: add the parts in ascending k order and store the tile
#pragma unroll 1
                for (int hc = 0; hc < MT * (BN / 32); ++hc) {
                    const int h = hc / (BN / 32), c = hc - h * (BN / 32);
                    const int row = h * BM + quad * 32 + lane;
                    const int m = tm * BMT + row;
                    const int n0 = n_base + c * 32;
                    if (m >= p.M || n0 >= p.N) continue;
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0.0f;
                    // two parts at a time: sixteen 16-byte loads in flight per thread, added in ascending k order
                    for (int cc = c_lo; cc <= c_hi; cc += 2) {
                        // a CTA that starts inside this tile holds the part in its first scratch tile, one that
                        // ends inside it (having started earlier) in its second
                        const int sl0 = SegIter::start_of(cc, p.sk_q, p.sk_r) >= u_lo ? 0 : 1;
                        const bool two = cc + 1 <= c_hi;
                        const float4* s0 = reinterpret_cast<const float4*>(p.sk_scratch + ((size_t)cc * 2 + sl0) * ((size_t)BMT * BN)) +
                                           (size_t)hc * 8 * 128 + quad * 32 + lane;
                        const float4* s1 = reinterpret_cast<const float4*>(p.sk_scratch + ((size_t)(cc + 1) * 2) * ((size_t)BMT * BN)) +
                                           (size_t)hc * 8 * 128 + quad * 32 + lane;   // a later part always starts inside the tile
                        float4 a4[8], b4[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) a4[j] = __ldcg(s0 + j * 128);
                        if (two) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) b4[j] = __ldcg(s1 + j * 128);
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            v[4 * j] += a4[j].x; v[4 * j + 1] += a4[j].y; v[4 * j + 2] += a4[j].z; v[4 * j + 3] += a4[j].w;
                        }
                        if (two) {
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                v[4 * j] += b4[j].x; v[4 * j + 1] += b4[j].y; v[4 * j + 2] += b4[j].z; v[4 * j + 3] += b4[j].w;
                            }
                        }
                    }
                    float* crow = p.C + (int64_t)m * p.N;
                    if (vec_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            if (n0 + j < p.N) {
                                float4 o4 = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                float4* dst = reinterpret_cast<float4*>(crow + n0 + j);
                                if (p.accumulate) {
                                    const float4 o = *dst;
                                    o4.x += o.x; o4.y += o.y; o4.z += o.z; o4.w += o.w;
                                }
                                *dst = o4;
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (n0 + j < p.N) crow[n0 + j] = p.accumulate ? crow[n0 + j] + v[j] : v[j];
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (threadIdx.x == 64) p.sk_tickets[t] = 0;   // ready for the next launch
                continue;
            }
#pragma unroll 1
            for (int hc = 0; hc < MT * (BN / 32); ++hc) {
                const int h = hc / (BN / 32), c = hc - h * (BN / 32);
                const int m = tm * BMT + h * BM + quad * 32 + lane;
                float* crow = p.C + (int64_t)m * p.N;
                uint32_t r[32];
                tmem_ld_32x32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)((acc + h) * BN + c * 32), r);
                tmem_ld_wait();
                const int n0 = n_base + c * 32;
                if (m < p.M) {
                    if (vec_ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            if (n0 + j < p.N) {
                                float4 v = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]),
                                                       __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                                float4* dst = reinterpret_cast<float4*>(crow + n0 + j);
                                if (p.accumulate) {
                                    float4 o = *dst;
                                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                                }
                                *dst = v;
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (n0 + j < p.N) {
                                float v = __uint_as_float(r[j]);
                                crow[n0 + j] = p.accumulate ? crow[n0 + j] + v : v;
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

    // teardown: everyone meets here, then the allocating warp returns the tensor memory
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// Self-test of the bounded wait every tensor-core kernel is built on: one CTA initialises an mbarrier
// that nothing will ever arrive on and waits for it with the given budget.  The wait must give up, the
// kernel must record MTL_ERR_TIMEOUT in the context's status word and return normally.
__global__ void k_bounded_wait_selftest(int32_t* status, uint64_t budget_ns, int32_t* waited_us) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint64_t t0 = globaltimer_ns();
        const bool ok = mbar_wait(&bar, 0, &abort_flag, budget_ns);
        if (waited_us) *waited_us = (int32_t)((globaltimer_ns() - t0) / 1000);
        if (!ok) atomicExch(status, MTL_ERR_TIMEOUT);
    }
    __syncthreads();
}

// hi = x rounded to tf32 (low 13 mantissa bits zero), lo = x - hi (exact in fp32)
__global__ void __launch_bounds__(256) k_split_tf32(float* __restrict__ hi, float* __restrict__ lo,
                                                    const float* __restrict__ x, int64_t n) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int64_t n4 = n >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    float4* h4 = reinterpret_cast<float4*>(hi);
    float4* l4 = reinterpret_cast<float4*>(lo);
    auto split = [](float v, float& h, float& l) {
        uint32_t u;
        asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
        h = __uint_as_float(u);
        l = v - h;
    };
    for (int64_t i = tid; i < n4; i += stride) {
        float4 v = x4[i], h, l;
        split(v.x, h.x, l.x); split(v.y, h.y, l.y); split(v.z, h.z, l.z); split(v.w, h.w, l.w);
        h4[i] = h;
        l4[i] = l;
    }
    for (int64_t i = (n4 << 2) + tid; i < n; i += stride) split(x[i], hi[i], lo[i]);
}

template <int BN, bool A_MN, bool B_MN, int MT>
int32_t launch_gemm(mtl_ctx* ctx, const CUtensorMap* maps, const GemmParams& p) {
    using C = Cfg<BN, MT>;
    auto kern = k_gemm_tf32<BN, A_MN, B_MN, MT>;
    MTL_CUDA(ctx, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    int tiles = ((p.M + BM * MT - 1) / (BM * MT)) * ((p.N + BN - 1) / BN);
    int grid = p.sk ? p.sk_grid : (tiles < ctx->sm_count ? tiles : ctx->sm_count);   // stream-K: equal shares of k-blocks
    {
        mtl_prof_scope prof(ctx, MTL_PROF_DOT_TC);
        kern<<<grid, kThreads, C::kSmemBytes, ctx->stream>>>(maps[0], maps[1], maps[2], maps[3], p);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

}  // namespace

int32_t mtl_encode_tmap(mtl_ctx* ctx, CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                        const uint64_t* strides_bytes, const uint32_t* box, int mode) {
    typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    if (!ctx->encode_tiled) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
            cudaGetLastError();
            return mtl_set_error(ctx, MTL_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
        }
        ctx->encode_tiled = fn;
    }
    cuuint64_t gdim[5];
    cuuint64_t gstr[4];
    cuuint32_t gbox[5];
    cuuint32_t estr[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        gbox[i] = box[i];
        estr[i] = 1;
        if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
    }
    CUresult r = ((encode_fn)ctx->encode_tiled)(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank,
                                               const_cast<void*>(base), gdim, gstr, gbox, estr,
                                               CU_TENSOR_MAP_INTERLEAVE_NONE,
                                               mode == 2 ? CU_TENSOR_MAP_SWIZZLE_NONE
                                               : mode == 1 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return mtl_set_error(ctx, MTL_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d)", (int)r, rank);
    return MTL_OK;
}

bool mtl_gemm_tc_supported(int64_t M, int64_t N, int64_t K, int transA, int transB, const float* A,
                           const float* B, const float* C) {
    if (M < 128 || N < 128 || K < 32) return false;
    if (M >= (1ll << 31) || N >= (1ll << 31) || K >= (1ll << 31)) return false;
    if ((((uintptr_t)A) | ((uintptr_t)B) | ((uintptr_t)C)) & 15u) return false;
    // global strides of a tensor map must be multiples of 16 bytes
    int64_t lda = transA ? M : K;  // contiguous extent of A's rows
    int64_t ldb = transB ? K : N;
    if ((lda % 4) || (ldb % 4)) return false;
    return true;
}

int32_t mtl_gemm_tc(mtl_ctx* ctx, float* C, const float* A, const float* B, int64_t M, int64_t N, int64_t K,
                    int transA, int transB, int accumulate, int x3) {
    if (!mtl_gemm_tc_supported(M, N, K, transA, transB, A, B, C))
        return mtl_set_error(ctx, MTL_ERR_UNSUPPORTED, "shape not supported by the tensor-core DOT kernel");
    int BN = N >= 256 ? 256 : 128;
    // few tiles: 128-column tiles put twice as many SMs to work (1024^3: 64 instead of 32)
    if (BN == 256 && ((M + 127) / 128) * ((N + 255) / 256) * 2 <= ctx->sm_count) BN = 128;
    if (ctx->tune.gemm_bn == 128 || (ctx->tune.gemm_bn == 256 && N >= 256)) BN = ctx->tune.gemm_bn;
    // 256-row tiles when they do not cost waves: a 256 x 256 tile takes about 1.67x a 128 x 256 one
    int MT = 1;
    if (BN == 256 && M >= 256) {
        const int64_t t1 = ((M + 127) / 128) * ((N + 255) / 256), t2 = ((M + 255) / 256) * ((N + 255) / 256);
        const int64_t w1 = (t1 + ctx->sm_count - 1) / ctx->sm_count, w2 = (t2 + ctx->sm_count - 1) / ctx->sm_count;
        if ((double)w2 * 1.67 < (double)w1 && K >= 512) MT = 2;
    }
    // Stream-K (see GemmParams::sk) is an opt-in (MANTLE_GEMM_SPLITK=1).  It keeps every SM busy whatever the
    // tile count, but each part of a split tile makes a trip through memory and only the four epilogue warps
    // of a CTA move it: measured on B200, 4096^3 took 0.273 ms with it against 0.205 ms with whole tiles
    // (1.73 waves), 2048^3 0.120 against 0.041 ms.  With it the tile is the largest one that still gives at
    // least a third as many tiles as SMs, so that a tile has about three parts at most.
    const int kb_units = (int)((K + BK - 1) / BK) * (x3 ? 3 : 1);
    int sk = 0;
    {
        const int64_t tiles = ((M + BM * MT - 1) / (BM * MT)) * ((N + BN - 1) / BN);
        const int64_t waves = (tiles + ctx->sm_count - 1) / ctx->sm_count;
        const double fill = (double)tiles / (double)(waves * ctx->sm_count);
        if (fill < 0.92 && kb_units >= 8 && ctx->tune.gemm_split_k >= 1) sk = 1;
        if (sk && ctx->tune.gemm_bn < 0 && ctx->tune.gemm_mt < 0) {
            const int64_t want = (ctx->sm_count + 2) / 3;
            const int64_t t22 = ((M + 255) / 256) * ((N + 255) / 256), t12 = ((M + 127) / 128) * ((N + 255) / 256);
            if (N >= 256 && M >= 256 && K >= 512 && t22 >= want) { BN = 256; MT = 2; }
            else if (N >= 256 && t12 >= want) { BN = 256; MT = 1; }
            else { BN = 128; MT = 1; }
        }
    }
    if (ctx->tune.gemm_mt == 1 || (ctx->tune.gemm_mt == 2 && BN == 256 && M >= 256)) MT = ctx->tune.gemm_mt;
    const int BMT = BM * MT;
    const float* a_src[2] = {A, nullptr};
    const float* b_src[2] = {B, nullptr};
    // scratch of the stream-K schedule: two tiles per CTA, behind the hi / lo operand copies
    const size_t sk_floats = sk ? (size_t)ctx->sm_count * 2 * BMT * BN : 0;
    float* sk_scratch = nullptr;
    if (sk && !x3) {
        void* ws;
        int32_t rc = mtl_workspace(ctx, sk_floats * sizeof(float), &ws);
        if (rc) return rc;
        sk_scratch = (float*)ws;
    }
    if (x3) {
        size_t na = (size_t)M * K, nb = (size_t)K * N;
        size_t na_pad = (na + 63) & ~(size_t)63, nb_pad = (nb + 63) & ~(size_t)63;
        void* ws;
        int32_t rc = mtl_workspace(ctx, (2 * na_pad + 2 * nb_pad + sk_floats) * sizeof(float), &ws);
        if (rc) return rc;
        float* w = (float*)ws;
        sk_scratch = w + 2 * na_pad + 2 * nb_pad;
        float *ahi = w, *alo = w + na_pad, *bhi = w + 2 * na_pad, *blo = w + 2 * na_pad + nb_pad;
        int g1 = mtl_grid_for((int64_t)(na + 3) / 4, 256, ctx->sm_count, 8);
        k_split_tf32<<<g1, 256, 0, ctx->stream>>>(ahi, alo, A, (int64_t)na);
        MTL_LAUNCHED(ctx);
        int g2 = mtl_grid_for((int64_t)(nb + 3) / 4, 256, ctx->sm_count, 8);
        k_split_tf32<<<g2, 256, 0, ctx->stream>>>(bhi, blo, B, (int64_t)nb);
        MTL_LAUNCHED(ctx);
        a_src[0] = ahi; a_src[1] = alo;
        b_src[0] = bhi; b_src[1] = blo;
    }
    // An MN-major operand stored [K, MN] can be fetched with ONE 3-D box per stage when MN is a
    // multiple of 32: dims {32, K, MN/32} with strides {row, 128 B}, box {32, BK, chunks}; its
    // shared-memory image [chunk][k][32] is exactly the chunked layout the descriptors expect.
    const bool no3d = !ctx->tune.gemm_3d_boxes;
    const int a3d = transA && (M % 32 == 0) && !no3d, b3d = !transB && (N % 32 == 0) && !no3d;
    CUtensorMap maps[4];
    for (int i = 0; i < 2; ++i) {
        const float* a = a_src[i] ? a_src[i] : a_src[0];
        const float* b = b_src[i] ? b_src[i] : b_src[0];
        uint64_t dims[3], strides[2];
        uint32_t box[3];
        int rank = 2;
        if (a3d) { dims[0] = 32; dims[1] = (uint64_t)K; dims[2] = (uint64_t)(M / 32); strides[0] = (uint64_t)M * 4; strides[1] = 128;
                   box[0] = 32; box[1] = BK; box[2] = (uint32_t)(BMT / 32); rank = 3; }
        else if (transA) { dims[0] = (uint64_t)M; dims[1] = (uint64_t)K; box[0] = 32; box[1] = BK; strides[0] = dims[0] * 4; }
        else             { dims[0] = (uint64_t)K; dims[1] = (uint64_t)M; box[0] = BK; box[1] = (uint32_t)BMT; strides[0] = dims[0] * 4; }
        int32_t rc = mtl_encode_tmap(ctx, &maps[i], a, rank, dims, strides, box, transA != 0);
        if (rc) return rc;
        rank = 2;
        if (b3d) { dims[0] = 32; dims[1] = (uint64_t)K; dims[2] = (uint64_t)(N / 32); strides[0] = (uint64_t)N * 4; strides[1] = 128;
                   box[0] = 32; box[1] = BK; box[2] = (uint32_t)(BN / 32); rank = 3; }
        else if (transB) { dims[0] = (uint64_t)K; dims[1] = (uint64_t)N; box[0] = BK; box[1] = (uint32_t)BN; strides[0] = dims[0] * 4; }
        else             { dims[0] = (uint64_t)N; dims[1] = (uint64_t)K; box[0] = 32; box[1] = BK; strides[0] = dims[0] * 4; }
        rc = mtl_encode_tmap(ctx, &maps[2 + i], b, rank, dims, strides, box, transB == 0);
        if (rc) return rc;
    }
    GemmParams p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.nseg = x3 ? 3 : 1;
    // small terms first: lo*hi, hi*lo, then hi*hi
    if (x3) { p.segA[0] = 1; p.segB[0] = 0; p.segA[1] = 0; p.segB[1] = 1; p.segA[2] = 0; p.segB[2] = 0; }
    else    { p.segA[0] = p.segA[1] = p.segA[2] = 0; p.segB[0] = p.segB[1] = p.segB[2] = 0; }
    p.C = C;
    p.accumulate = accumulate ? 1 : 0;
    p.status = ctx->dev_status;
    p.stages = MT == 2 ? 3 : (BN == 256 ? 4 : 6);
    p.a3d = a3d;
    p.b3d = b3d;
    p.sk = 0; p.sk_grid = 0; p.sk_q = 0; p.sk_r = 0; p.sk_scratch = nullptr; p.sk_tickets = ctx->tickets;
    {
        const int64_t tiles = ((M + BMT - 1) / BMT) * ((N + BN - 1) / BN);
        const int64_t units = tiles * kb_units;
        int64_t grid = ctx->sm_count;
        if (grid > tiles * 4) grid = tiles * 4;
        if (sk && tiles <= 8190 && grid > tiles / 2 && units >= grid * 2) {
            p.sk = 1;
            p.sk_grid = (int)grid;
            p.sk_q = units / grid;
            p.sk_r = units % grid;
            p.sk_scratch = sk_scratch;
        }
    }
    if (ctx->tune.gemm_stages >= 1 && ctx->tune.gemm_stages <= p.stages) p.stages = ctx->tune.gemm_stages;
    const bool a_mn = transA != 0, b_mn = transB == 0;
#define MTL_DISPATCH(BN_, MT_)                                                                \
    if (a_mn && b_mn) return launch_gemm<BN_, true, true, MT_>(ctx, maps, p);                \
    if (a_mn && !b_mn) return launch_gemm<BN_, true, false, MT_>(ctx, maps, p);              \
    if (!a_mn && b_mn) return launch_gemm<BN_, false, true, MT_>(ctx, maps, p);              \
    return launch_gemm<BN_, false, false, MT_>(ctx, maps, p);
    if (BN == 256 && MT == 2) { MTL_DISPATCH(256, 2) }
    if (BN == 256) { MTL_DISPATCH(256, 1) }
    MTL_DISPATCH(128, 1)
#undef MTL_DISPATCH
}

extern "C" {

int32_t mtl_selftest_bounded_wait(mtl_ctx* ctx, int32_t budget_us, int32_t* waited_us) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, budget_us >= 1 && budget_us <= 1000000, "budget must be 1 .. 1000000 microseconds");
    MTL_REQUIRE(ctx, !ctx->capturing, "the self-test reads its result back and cannot be captured");
    int32_t* d_waited = nullptr;
    void* ws;
    int32_t rc = mtl_workspace(ctx, 256, &ws);
    if (rc) return rc;
    d_waited = (int32_t*)ws;
    k_bounded_wait_selftest<<<1, 32, 0, ctx->stream>>>(ctx->dev_status, (uint64_t)budget_us * 1000ull, d_waited);
    MTL_LAUNCHED(ctx);
    if (waited_us) {
        MTL_CUDA(ctx, cudaMemcpyAsync(waited_us, d_waited, 4, cudaMemcpyDeviceToHost, ctx->stream));
        MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    return MTL_OK;
}

int32_t mtl_dot_fwd(mtl_ctx* ctx, float* C, const float* A, const float* B, int64_t M, int64_t K, int64_t N) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, C && A && B, "null pointer in mtl_dot_fwd");
    MTL_REQUIRE(ctx, M >= 1 && K >= 1 && N >= 1, "DOT extents must be positive");
    if (ctx->math_mode != MTL_MATH_FP32 && mtl_gemm_tc_supported(M, N, K, 0, 0, A, B, C))
        return mtl_gemm_tc(ctx, C, A, B, M, N, K, 0, 0, 0, ctx->math_mode == MTL_MATH_TF32X3);
    if (ctx->math_mode != MTL_MATH_FP32 && mtl_gemm_thin_supported(M, N, K, 0, 0))
        return mtl_gemm_thin(ctx, C, A, B, M, N, K, 0, 0);
    return mtl_gemm_simt(ctx, C, A, B, M, N, K, 0, 0, 0);
}

int32_t mtl_dot_bwd(mtl_ctx* ctx, int32_t tensor_id, float* grad, const float* ug, const float* A,
                    const float* B, int64_t M, int64_t K, int64_t N, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, tensor_id == 0 || tensor_id == 1, "tensor_id must be 0 or 1");
    MTL_REQUIRE(ctx, grad && ug, "null pointer in mtl_dot_bwd");
    MTL_REQUIRE(ctx, M >= 1 && K >= 1 && N >= 1, "DOT extents must be positive");
    const bool tc = ctx->math_mode != MTL_MATH_FP32;
    const int x3 = ctx->math_mode == MTL_MATH_TF32X3;
    if (tensor_id == 0) {
        // grad[M,K] = ug[M,N] . B[K,N]^T : product extents (M, K, N)
        MTL_REQUIRE(ctx, B, "dA needs B");
        if (tc && mtl_gemm_tc_supported(M, K, N, 0, 1, ug, B, grad))
            return mtl_gemm_tc(ctx, grad, ug, B, M, K, N, 0, 1, accumulate, x3);
        return mtl_gemm_simt(ctx, grad, ug, B, M, K, N, 0, 1, accumulate);
    }
    // grad[K,N] = A[M,K]^T . ug[M,N] : product extents (K, N, M)
    MTL_REQUIRE(ctx, A, "dB needs A");
    if (tc && mtl_gemm_tc_supported(K, N, M, 1, 0, A, ug, grad))
        return mtl_gemm_tc(ctx, grad, A, ug, K, N, M, 1, 0, accumulate, x3);
    if (tc && mtl_gemm_thin_supported(K, N, M, 1, 0)) return mtl_gemm_thin(ctx, grad, A, ug, K, N, M, 1, accumulate);
    return mtl_gemm_simt(ctx, grad, A, ug, K, N, M, 1, 0, accumulate);
}

}  // extern "C"
