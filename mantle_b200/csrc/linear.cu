// nn.Linear as the reference builds it -- a DOT node followed by an ADD of the bias
// (mantle/nn/layers/linear.mojo:25-46) -- for layers with at most 16 outputs (classifier heads), as
// ONE launch forward and ONE launch backward.  Such products are tiny in arithmetic and bound by
// streaming the [M, K] activations once; run as separate operator calls they cost eight launches a
// step (product, fold of the k-slices, bias add; bias gradient in two, the two operand gradients,
// another fold), which at small batches is most of their time.
//
//   forward   C[M,N] (+)= A[M,K] . B[K,N] + bias[N]
//             DOT.forward (basics.mojo:230-237) then ADD.forward with a broadcast bias (basics.mojo:21-43)
//   backward  dA[M,K] (+)= ug . B^T, dB[K,N] (+)= A^T . ug      DOT.backward (basics.mojo:240-257)
//             dbias[N] (+)= column sums of ug                   ADD.backward + un-broadcast (basics.mojo:46-66,
//                                                               tensorutils.mojo:455-487)
//
// Sums over k (forward) and over the batch (dB) are split over many blocks so that the GPU is full at
// any batch size; the slices are folded IN THE SAME LAUNCH, in ascending slice order, by whichever
// block of a row group finishes last (a ticket counter per row group), so results do not depend on
// the order in which blocks run.  The forward product runs on the tensor cores' warp-level instruction with
// every operand split into two TF32 parts (three products, fp32 accumulation: within a few ulp of fp32), the
// gradients as fp32 FMA on CUDA cores; sums are re-associated with respect to the reference's ascending chain
// (compared at rtol = atol = 1e-5), so MTL_MATH_FP32, which promises that chain bit for bit, takes the
// separate operator kernels instead.
#include "common.cuh"

namespace {

constexpr int kTicketsFwd = 4096; // ticket slots [0, 4096) forward row groups, [4096, 8192) dB column groups

// ------------------------------------------------------------------ forward --------------------
// The sums over k are done by the tensor cores' warp-level instruction
// (mma.sync m16n8k8, TF32 operands, fp32 accumulation), which needs no exchange between lanes: a warp owns 16
// rows of A, a block of eight warps 128 rows and one k slice.  Each operand is split into a TF32 head and a
// TF32 tail and three products are accumulated (head x head, head x tail, tail x head), which keeps the
// result within a few ulp of the fp32 product; the kernel is bound by streaming A, not by arithmetic.
// The reduction order inside a step is free, so the k positions of a fragment are chosen to make the loads
// wide: lane (g, t) -- g = lane / 4, t = lane % 4 -- reads rows g and g + 8 at k0 + 4 t .. + 3 and at
// k0 + 16 + 4 t .. + 3 (16-byte loads; eight lanes cover 128 contiguous bytes of a row), and the j-th of four
// instructions takes element j of each piece; the matching rows of B are k0 + 4 t + j and k0 + 16 + 4 t + j.
// B's rows sit in shared memory with a stride of 18 floats: the 32 lanes of a fragment read hit 32 banks.
__device__ __forceinline__ uint32_t tf32_head(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void mma_tf32_16x8x8(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
constexpr int kMmaKC = 256;      // largest k slice of a block
constexpr int kMmaBS = 18;       // floats between rows of B in shared memory

template <int NT>   // n8 tiles: 1 for N <= 8, 2 for N <= 16
__global__ void __launch_bounds__(256, 2) k_linear_fwd_mma(float* __restrict__ C, float* __restrict__ partial,
                                                           int32_t* __restrict__ tickets, const float* __restrict__ A,
                                                           const float* __restrict__ B, const float* __restrict__ bias,
                                                           int M, int N, int K, int kc, int accumulate) {
    __shared__ float b_s[kMmaKC * kMmaBS];
    __shared__ int s_last;
    mtl_pdl_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int k_begin = blockIdx.y * kc;
    const int kn = min(kc, K - k_begin);          // a multiple of four (K and kc are)
    const int m0 = blockIdx.x * 128 + warp * 16;  // rows past M load zeros and store nothing
    const float* row_lo = A + (int64_t)(m0 + g) * K + k_begin;
    const float* row_hi = A + (int64_t)(m0 + g + 8) * K + k_begin;
    const bool lo_ok = m0 + g < M, hi_ok = m0 + g + 8 < M;
    // The operands of A travel in batches of two steps (64 values of k): two batches are in flight before
    // anything else, and the batch after next is asked for before a batch is multiplied.
    float4 pa[2][2][4];                           // [buffer][step][row g | row g+8 | row g (+16) | row g+8 (+16)]
    auto fetch = [&](float4 (&dst)[2][4], int s0) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            const int k0 = (s0 + s) * 32 + 4 * t;
            const float4 z = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            dst[s][0] = (lo_ok && k0 < kn) ? __ldg(reinterpret_cast<const float4*>(row_lo + k0)) : z;
            dst[s][1] = (hi_ok && k0 < kn) ? __ldg(reinterpret_cast<const float4*>(row_hi + k0)) : z;
            dst[s][2] = (lo_ok && k0 + 16 < kn) ? __ldg(reinterpret_cast<const float4*>(row_lo + k0 + 16)) : z;
            dst[s][3] = (hi_ok && k0 + 16 < kn) ? __ldg(reinterpret_cast<const float4*>(row_hi + k0 + 16)) : z;
        }
    };
    fetch(pa[0], 0);
    fetch(pa[1], 2);
    // the slice's rows of B, zero beyond column N
    for (int i = threadIdx.x; i < kMmaKC * kMmaBS; i += 256) b_s[i] = 0.0f;
    __syncthreads();
    {
        const int total = kn * N;                 // a multiple of four
        const float4* bsrc = reinterpret_cast<const float4*>(B + (int64_t)k_begin * N);
        for (int f = threadIdx.x; f * 4 < total; f += 256) {
            const float4 v = __ldg(bsrc + f);
            const float pv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int idx = f * 4 + e;
                const int kk = idx / N, j = idx - kk * N;
                b_s[kk * kMmaBS + j] = pv[e];
            }
        }
    }
    __syncthreads();
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    const int steps = (kn + 31) / 32;
    auto multiply = [&](const float4 (&src)[2][4], int s0) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            if (s0 + s < steps) {
                const int kb = (s0 + s) * 32 + 4 * t;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float av[4] = {j == 0 ? src[s][0].x : j == 1 ? src[s][0].y : j == 2 ? src[s][0].z : src[s][0].w,
                                         j == 0 ? src[s][1].x : j == 1 ? src[s][1].y : j == 2 ? src[s][1].z : src[s][1].w,
                                         j == 0 ? src[s][2].x : j == 1 ? src[s][2].y : j == 2 ? src[s][2].z : src[s][2].w,
                                         j == 0 ? src[s][3].x : j == 1 ? src[s][3].y : j == 2 ? src[s][3].z : src[s][3].w};
                    uint32_t ah[4], al[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        ah[i] = tf32_head(av[i]);
                        al[i] = tf32_head(av[i] - __uint_as_float(ah[i]));
                    }
#pragma unroll
                    for (int n = 0; n < NT; ++n) {
                        const float b0 = b_s[(kb + j) * kMmaBS + n * 8 + g];
                        const float b1 = b_s[(kb + 16 + j) * kMmaBS + n * 8 + g];
                        const uint32_t b0h = tf32_head(b0), b1h = tf32_head(b1);
                        const uint32_t b0l = tf32_head(b0 - __uint_as_float(b0h)), b1l = tf32_head(b1 - __uint_as_float(b1h));
                        mma_tf32_16x8x8(acc[n], al, b0h, b1h);      // small terms first
                        mma_tf32_16x8x8(acc[n], ah, b0l, b1l);
                        mma_tf32_16x8x8(acc[n], ah, b0h, b1h);
                    }
                }
            }
        }
    };
    for (int s0 = 0; s0 < steps; s0 += 4) {
        float4 cur[2][4];
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int i = 0; i < 4; ++i) cur[s][i] = pa[0][s][i];
        if (s0 + 4 < steps) fetch(pa[0], s0 + 4);
        multiply(cur, s0);
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int i = 0; i < 4; ++i) cur[s][i] = pa[1][s][i];
        if (s0 + 6 < steps) fetch(pa[1], s0 + 6);
        multiply(cur, s0 + 2);
    }
    // accumulator element (row g [+8], column 2 t [+1]) of every n8 tile goes to this slice's partial result
    float* out = partial + (int64_t)blockIdx.y * M * N;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        const int c0 = n * 8 + 2 * t;
        if (lo_ok) {
            if (c0 < N) out[(int64_t)(m0 + g) * N + c0] = acc[n][0];
            if (c0 + 1 < N) out[(int64_t)(m0 + g) * N + c0 + 1] = acc[n][1];
        }
        if (hi_ok) {
            if (c0 < N) out[(int64_t)(m0 + g + 8) * N + c0] = acc[n][2];
            if (c0 + 1 < N) out[(int64_t)(m0 + g + 8) * N + c0 + 1] = acc[n][3];
        }
    }
    // ---- the block that finishes last for this group of 128 rows folds the k slices, in ascending order
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&tickets[blockIdx.x], 1) == (int)gridDim.y - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int nsplit = gridDim.y;
    const int rows = min(128, M - (int)blockIdx.x * 128);
    const int64_t base = (int64_t)blockIdx.x * 128 * N;      // the group's rows are rows * N contiguous floats per slice
    const int64_t slice = (int64_t)M * N;
    if ((slice & 3) == 0 && ((rows * N) & 3) == 0) {
        // 16-byte pieces, eight slices in flight per thread, slices added in ascending order
        const float4* p4 = reinterpret_cast<const float4*>(partial + base);
        const int64_t slice4 = slice >> 2;
        for (int i4 = threadIdx.x; i4 < (rows * N) >> 2; i4 += 256) {
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            int sp = 0;
            for (; sp + 8 <= nsplit; sp += 8) {
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = __ldcg(p4 + (int64_t)(sp + u) * slice4 + i4);
#pragma unroll
                for (int u = 0; u < 8; ++u) { sum.x += v[u].x; sum.y += v[u].y; sum.z += v[u].z; sum.w += v[u].w; }
            }
            for (; sp < nsplit; ++sp) {
                const float4 v = __ldcg(p4 + (int64_t)sp * slice4 + i4);
                sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
            }
            const float sv[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int idx = i4 * 4 + e;
                const int col = idx % N;
                float r = sv[e];
                if (bias) r += __ldg(bias + col);     // ADD.forward after DOT.forward
                float* c = C + base + idx;
                *c = accumulate ? *c + r : r;
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < rows * N; idx += 256) {
            const int col = idx % N;
            float sum = 0.0f;
            for (int sp = 0; sp < nsplit; ++sp) sum += __ldcg(partial + (int64_t)sp * slice + base + idx);
            if (bias) sum += __ldg(bias + col);       // ADD.forward after DOT.forward
            float* c = C + base + idx;
            *c = accumulate ? *c + sum : sum;
        }
    }
    if (threadIdx.x == 0) tickets[blockIdx.x] = 0;   // ready for the next launch
}

// ------------------------------------------------------------------ backward -------------------
struct LinBwd {
    float* dA; float* dB; float* dbias;
    const float* ug; const float* A; const float* B;
    float* partial;          // [msplit][K][N] slices of dB
    int32_t* tickets;        // one per group of 256 columns of A (= rows of dB)
    int M, N, K;
    int acc_da, acc_db, acc_dbias;
    int n_da_blocks, da_kt, da_rows;  // role dA: blocks, tiles of 1024 along K, rows of ug per block
    int n_db_blocks, kgroups, msplit, rows_per_split;   // role dB
};

// dA[m, k] (+)= sum_j ug[m, j] * B[k, j].  A block owns da_rows rows of ug and 1024 values of k.  Its
// slice of B (1024 x N floats, contiguous) is read once with coalesced loads into shared memory, row
// stride N | 1 floats; thread t then keeps rows k0 + 4 t .. 4 t + 3 in registers and walks the rows of ug,
// storing four consecutive values of a row of dA at a time (a warp's store covers 512 contiguous bytes).
constexpr int kDaKT = 1024;
template <int NP>
__device__ __forceinline__ void role_da(const LinBwd& p, int b, float* smem) {
    const int kt = b % p.da_kt, mt = b / p.da_kt;
    const int m0 = mt * p.da_rows;
    const int k_base = kt * kDaKT;
    const int kn = min(kDaKT, p.K - k_base);
    const int ws = p.N | 1;
    float* w_s = smem;                                    // [1024][N | 1]
    float* ug_s = smem + kDaKT * ws;                      // [da_rows][16]
    // the slice is kn * N contiguous floats (a multiple of four, 16-byte aligned): every thread's 16-byte
    // pieces are in flight together
    {
        const float4* wsrc = reinterpret_cast<const float4*>(p.B + (int64_t)k_base * p.N);
        const int total = kn * p.N;
        constexpr int kPieces = (kDaKT * NP / 4 + 255) / 256;
        float4 piece[kPieces];
#pragma unroll
        for (int t = 0; t < kPieces; ++t) {
            const int f = t * 256 + (int)threadIdx.x;
            piece[t] = f * 4 < total ? __ldg(wsrc + f) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int t = 0; t < kPieces; ++t) {
            const int f = t * 256 + (int)threadIdx.x;
            if (f * 4 < total) {
                const float pv[4] = {piece[t].x, piece[t].y, piece[t].z, piece[t].w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int idx = f * 4 + e;
                    const int kk = idx / p.N, j = idx - kk * p.N;
                    w_s[kk * ws + j] = pv[e];
                }
            }
        }
    }
    for (int i = threadIdx.x; i < p.da_rows * 16; i += 256) {
        const int r = i >> 4, j = i & 15;
        ug_s[i] = (m0 + r < p.M && j < p.N) ? __ldg(p.ug + (int64_t)(m0 + r) * p.N + j) : 0.0f;
    }
    __syncthreads();
    float w[4][NP];
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        const int kl = threadIdx.x * 4 + kk;
#pragma unroll
        for (int j = 0; j < NP; ++j) w[kk][j] = (kl < kn && j < p.N) ? w_s[kl * ws + j] : 0.0f;
    }
    const int rows = min(p.da_rows, p.M - m0);
#pragma unroll 2
    for (int r = 0; r < rows; ++r) {
        float o[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int j = 0; j < NP; ++j) {
            const float u = ug_s[r * 16 + j];             // ascending j, like dot_transpose_t2's chain
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) o[kk] = fmaf(u, w[kk][j], o[kk]);
        }
        if ((int)threadIdx.x * 4 < kn) {                  // kn is a multiple of four
            float4* dst = reinterpret_cast<float4*>(p.dA + (int64_t)(m0 + r) * p.K + k_base + threadIdx.x * 4);
            float4 v = make_float4(o[0], o[1], o[2], o[3]);
            if (p.acc_da) {
                const float4 old = *dst;
                v.x += old.x; v.y += old.y; v.z += old.z; v.w += old.w;
            }
            *dst = v;
        }
    }
}

// dB[k, j] (+)= sum_m A[m, k] * ug[m, j]: one thread per k, a slice of the batch per block; the block
// that finishes last for its 256 values of k folds the slices in ascending order.
template <int NP>
__device__ __forceinline__ void role_db(const LinBwd& p, int b, float* smem, int* s_last) {
    const int kg = b % p.kgroups, sp = b / p.kgroups;
    const int k = kg * 256 + threadIdx.x;
    const int m_begin = sp * p.rows_per_split;
    const int m_end = min(p.M, m_begin + p.rows_per_split);
    float acc[NP];
#pragma unroll
    for (int j = 0; j < NP; ++j) acc[j] = 0.0f;
    float* ug_s = smem;                                   // [64][16]
    for (int mb = m_begin; mb < m_end; mb += 64) {
        __syncthreads();
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i >> 4, j = i & 15;
            ug_s[i] = (mb + r < m_end && j < p.N) ? __ldg(p.ug + (int64_t)(mb + r) * p.N + j) : 0.0f;
        }
        __syncthreads();
        if (k < p.K) {
            const int mn = min(64, m_end - mb);
            for (int r0 = 0; r0 < mn; r0 += 32) {         // 32 loads of A in flight: two memory round trips per 64 rows
                float a[32];
#pragma unroll
                for (int u = 0; u < 32; ++u) a[u] = r0 + u < mn ? __ldg(p.A + (int64_t)(mb + r0 + u) * p.K + k) : 0.0f;
#pragma unroll
                for (int u = 0; u < 32; ++u) {
#pragma unroll
                    for (int q = 0; q < NP / 4; ++q) {
                        const float4 t = *reinterpret_cast<const float4*>(ug_s + (r0 + u) * 16 + 4 * q);
                        acc[4 * q] = fmaf(a[u], t.x, acc[4 * q]);
                        acc[4 * q + 1] = fmaf(a[u], t.y, acc[4 * q + 1]);
                        acc[4 * q + 2] = fmaf(a[u], t.z, acc[4 * q + 2]);
                        acc[4 * q + 3] = fmaf(a[u], t.w, acc[4 * q + 3]);
                    }
                }
            }
        }
    }
    if (k < p.K) {
        float* out = p.partial + ((int64_t)sp * p.K + k) * p.N;
#pragma unroll
        for (int j = 0; j < NP; ++j)
            if (j < p.N) out[j] = acc[j];
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *s_last = atomicAdd(&p.tickets[kg], 1) == p.msplit - 1;
    __syncthreads();
    if (!*s_last) return;
    __threadfence();
    const int kn = min(256, p.K - kg * 256);
    const int64_t slice = (int64_t)p.K * p.N, base = (int64_t)kg * 256 * p.N;
    if ((slice & 3) == 0 && ((kn * p.N) & 3) == 0 && (reinterpret_cast<uintptr_t>(p.dB) & 15u) == 0) {
        // 16-byte pieces, eight slices in flight per thread, slices added in ascending order
        const float4* p4 = reinterpret_cast<const float4*>(p.partial + base);
        float4* d4 = reinterpret_cast<float4*>(p.dB + base);
        const int64_t slice4 = slice >> 2;
        for (int i4 = threadIdx.x; i4 < (kn * p.N) >> 2; i4 += 256) {
            float4 s = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            int q = 0;
            for (; q + 8 <= p.msplit; q += 8) {
                float4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = __ldcg(p4 + (int64_t)(q + u) * slice4 + i4);
#pragma unroll
                for (int u = 0; u < 8; ++u) { s.x += v[u].x; s.y += v[u].y; s.z += v[u].z; s.w += v[u].w; }
            }
            for (; q < p.msplit; ++q) {
                const float4 v = __ldcg(p4 + (int64_t)q * slice4 + i4);
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
            if (p.acc_db) {
                const float4 old = d4[i4];
                s.x += old.x; s.y += old.y; s.z += old.z; s.w += old.w;
            }
            d4[i4] = s;
        }
    } else {
        for (int idx = threadIdx.x; idx < kn * p.N; idx += 256) {   // consecutive threads, consecutive floats
            const int64_t off = base + idx;
            float s = 0.0f;
            for (int q = 0; q < p.msplit; ++q) s += __ldcg(p.partial + (int64_t)q * slice + off);
            p.dB[off] = p.acc_db ? p.dB[off] + s : s;
        }
    }
    if (threadIdx.x == 0) p.tickets[kg] = 0;
}

// dbias[j] (+)= sum_m ug[m, j]: one block, sixteen row phases per column, folded in a fixed order.
__device__ __forceinline__ void role_dbias(const LinBwd& p, float* smem) {
    const int j = threadIdx.x & 15, ph = threadIdx.x >> 4;   // 16 phases
    float s = 0.0f;
    if (j < p.N)
        for (int m = ph; m < p.M; m += 16) s += __ldg(p.ug + (int64_t)m * p.N + j);
    smem[ph * 16 + j] = s;
    __syncthreads();
    if (threadIdx.x < p.N) {
        float t = 0.0f;
#pragma unroll
        for (int q = 0; q < 16; ++q) t += smem[q * 16 + threadIdx.x];
        p.dbias[threadIdx.x] = p.acc_dbias ? p.dbias[threadIdx.x] + t : t;
    }
}

template <int NP>
__global__ void __launch_bounds__(256) k_linear_bwd(LinBwd p) {
    extern __shared__ __align__(16) float smem[];   // role dA: B slice + rows of ug; role dB: 64 rows of ug
    __shared__ int s_last;
    mtl_pdl_sync();
    int b = blockIdx.x;
    if (b < p.n_db_blocks) { role_db<NP>(p, b, smem, &s_last); return; }      // the longest role first
    b -= p.n_db_blocks;
    if (b < p.n_da_blocks) { role_da<NP>(p, b, smem); return; }
    role_dbias(p, smem);
}

bool linear_supported(mtl_ctx* ctx, int64_t M, int64_t K, int64_t N) {
    return ctx->math_mode != MTL_MATH_FP32 && N >= 1 && N <= 16 && M >= 1 && K >= 1 && M <= (int64_t)kTicketsFwd * 32 &&
           K <= (int64_t)kTicketsFwd * 256 && M * K < (1ll << 40);
}

}  // namespace

extern "C" {

int32_t mtl_linear_fwd(mtl_ctx* ctx, float* C, const float* A, const float* B, const float* bias, int64_t M, int64_t K,
                       int64_t N) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, C && A && B, "null pointer in mtl_linear_fwd");
    MTL_REQUIRE(ctx, M >= 1 && K >= 1 && N >= 1, "Linear extents must be positive");
    if (!linear_supported(ctx, M, K, N) || K % 4 != 0 || ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B)) & 15u)) {   // 16-byte loads
        // the reference's two operator calls, one after the other
        int32_t rc = mtl_dot_fwd(ctx, C, A, B, M, K, N);
        if (rc || !bias) return rc;
        const int64_t cs[2] = {M, N}, bs[1] = {N};
        return mtl_binary_fwd(ctx, MTL_OP_ADD, C, C, bias, 2, cs, 1, bs);
    }
    // 128 rows and one k slice per block.  Shorter slices mean more blocks but also more slices for the last
    // block of a row group to fold (measured at 256 rows: 98 slices of 64 cost more in the fold than they
    // gain in parallelism), so slices shrink only until half the SMs have a block.
    const int rb = (int)((M + 127) / 128);
    int kc = kMmaKC;
    while (kc > 64 && (int64_t)rb * ((K + kc - 1) / kc) < ctx->sm_count / 2) kc >>= 1;
    const int nsplit = (int)((K + kc - 1) / kc);
    void* ws;
    int32_t rc = mtl_workspace(ctx, (size_t)nsplit * M * N * 4, &ws);
    if (rc) return rc;
    dim3 grid((unsigned)rb, (unsigned)nsplit);
    MTL_REQUIRE(ctx, nsplit <= 65535, "Linear: reduction too long");
    if (N <= 8)
        mtl_launch_pdl(ctx, k_linear_fwd_mma<1>, grid, dim3(256), (size_t)0, C, (float*)ws, ctx->tickets, A, B, bias, (int)M, (int)N, (int)K, kc, 0);
    else
        mtl_launch_pdl(ctx, k_linear_fwd_mma<2>, grid, dim3(256), (size_t)0, C, (float*)ws, ctx->tickets, A, B, bias, (int)M, (int)N, (int)K, kc, 0);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_linear_bwd(mtl_ctx* ctx, float* dA, float* dB, float* dbias, const float* ug, const float* A, const float* B,
                       int64_t M, int64_t K, int64_t N, int32_t acc_da, int32_t acc_db, int32_t acc_dbias) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, ug, "null upper gradient in mtl_linear_bwd");
    MTL_REQUIRE(ctx, M >= 1 && K >= 1 && N >= 1, "Linear extents must be positive");
    MTL_REQUIRE(ctx, (!dA || B) && (!dB || A), "mtl_linear_bwd: dA needs B and dB needs A");
    if (!dA && !dB && !dbias) return MTL_OK;
    const bool vec_ok = K % 4 == 0 && ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(dA) |
                                        reinterpret_cast<uintptr_t>(B)) & 15u) == 0;   // 16-byte accesses
    if (!linear_supported(ctx, M, K, N) || !vec_ok) {
        int32_t rc = MTL_OK;
        const int64_t cs[2] = {M, N}, bs[1] = {N};
        if (dbias) rc = mtl_binary_bwd(ctx, MTL_OP_ADD, 1, dbias, ug, ug, dbias, 2, cs, 1, bs, acc_dbias);
        if (!rc && dB) rc = mtl_dot_bwd(ctx, 1, dB, ug, A, B, M, K, N, acc_db);
        if (!rc && dA) rc = mtl_dot_bwd(ctx, 0, dA, ug, A, B, M, K, N, acc_da);
        return rc;
    }
    LinBwd p;
    p.dA = dA; p.dB = dB; p.dbias = dbias; p.ug = ug; p.A = A; p.B = B;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.acc_da = acc_da ? 1 : 0; p.acc_db = acc_db ? 1 : 0; p.acc_dbias = acc_dbias ? 1 : 0;
    p.da_kt = (int)((K + kDaKT - 1) / kDaKT);
    // rows of ug per block: 32 amortise the block's slice of B; fewer when that would leave SMs without a block
    p.da_rows = 32;
    while (p.da_rows > 4 && ((M + p.da_rows - 1) / p.da_rows) * p.da_kt < 2ll * ctx->sm_count) p.da_rows >>= 1;
    p.n_da_blocks = dA ? (int)((M + p.da_rows - 1) / p.da_rows) * p.da_kt : 0;
    p.kgroups = (int)((K + 255) / 256);
    p.msplit = 0; p.rows_per_split = 0; p.n_db_blocks = 0; p.partial = nullptr;
    p.tickets = ctx->tickets + kTicketsFwd;
    if (dB) {
        int want = (8 * ctx->sm_count + p.kgroups - 1) / p.kgroups;      // slices of the batch
        int64_t rows = (M + want - 1) / want;
        rows = (rows + 31) / 32 * 32;
        p.rows_per_split = (int)rows;
        p.msplit = (int)((M + rows - 1) / rows);
        p.n_db_blocks = p.kgroups * p.msplit;
        void* ws;
        int32_t rc = mtl_workspace(ctx, (size_t)p.msplit * K * N * 4, &ws);
        if (rc) return rc;
        p.partial = (float*)ws;
    }
    const int blocks = p.n_db_blocks + p.n_da_blocks + (dbias ? 1 : 0);
    size_t smem_bytes = (size_t)64 * 16 * 4;
    if (dA && (size_t)(kDaKT * ((int)N | 1) + 32 * 16) * 4 > smem_bytes) smem_bytes = (size_t)(kDaKT * ((int)N | 1) + 32 * 16) * 4;
#define MTL_LIN_BWD(NP_)                                                                                              \
    do {                                                                                                              \
        MTL_CUDA(ctx, cudaFuncSetAttribute(k_linear_bwd<NP_>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                                           (int)((kDaKT * 17 + 32 * 16) * 4)));                                       \
        mtl_launch_pdl(ctx, k_linear_bwd<NP_>, dim3((unsigned)blocks), dim3(256), smem_bytes, p);                     \
    } while (0)
    if (N <= 4) MTL_LIN_BWD(4);
    else if (N <= 8) MTL_LIN_BWD(8);
    else if (N <= 12) MTL_LIN_BWD(12);
    else MTL_LIN_BWD(16);
#undef MTL_LIN_BWD
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

}  // extern "C"
