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
// the order in which blocks run.  Arithmetic is fp32 FMA on CUDA cores; the k sum is re-associated
// with respect to the reference's ascending chain (compared at rtol = atol = 1e-5), so MTL_MATH_FP32,
// which promises that chain bit for bit, takes the separate operator kernels instead.
#include "common.cuh"

namespace {

constexpr int kKC = 256;          // largest k extent of one forward block (rows of B staged in shared memory)
constexpr int kTicketsFwd = 4096; // ticket slots [0, 4096) forward row groups, [4096, 8192) dB column groups

// ------------------------------------------------------------------ forward --------------------
// A block of eight warps owns 32 rows of A (four per warp) and one k slice of at most 256.  Every thread
// first asks for ALL its operands -- eight 16-byte loads of A and its share of the block's rows of B (kn * N
// contiguous floats, fetched as 16-byte pieces) -- so a block pays the memory latency once; two blocks share
// an SM.  Lane l of a warp holds k = 4 * (32 u + l) + e (u < 2, e < 4) of its four rows; the rows of B sit in
// shared memory in the order (e, 32 u + l), padded to an odd number of 16-byte units, so that the lanes of a
// warp read different banks.
template <int NQ>
__global__ void __launch_bounds__(256, 2) k_linear_fwd(float* __restrict__ C, float* __restrict__ partial,
                                                       int32_t* __restrict__ tickets, const float* __restrict__ A,
                                                       const float* __restrict__ B, const float* __restrict__ bias,
                                                       int M, int N, int K, int kc, int accumulate) {
    constexpr int NP = 4 * NQ;
    constexpr int RU = NQ | 1;
    constexpr int kPieces = (kKC * NP / 4 + 255) / 256;
    constexpr int kRed = (8 * 32 * (NP + 1) + 3) / 4;              // float4 units the row reduction below needs
    __shared__ float4 b_s[kKC * RU > kRed ? kKC * RU : kRed];
    __shared__ int s_last;
    mtl_pdl_sync();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_begin = blockIdx.y * kc;
    const int kn = min(kc, K - k_begin);          // a multiple of four (K and kc are)
    const int m0 = (blockIdx.x * 8 + warp) * 4;   // rows past M load zeros and store nothing
    float4 a[2][4];
    const float* a0 = A + (int64_t)m0 * K + k_begin;
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int kk = (u * 32 + lane) * 4;
            a[u][r] = (kk < kn && m0 + r < M) ? __ldg(reinterpret_cast<const float4*>(a0 + (int64_t)r * K + kk))
                                              : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
    const int total = kn * N;                     // a multiple of four
    const float4* bsrc = reinterpret_cast<const float4*>(B + (int64_t)k_begin * N);
    float4 piece[kPieces];
#pragma unroll
    for (int t = 0; t < kPieces; ++t) {
        const int f = t * 256 + (int)threadIdx.x;
        piece[t] = f * 4 < total ? __ldg(bsrc + f) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    float* b_f = reinterpret_cast<float*>(b_s);
    if (N < NP) {                                  // the columns past N must read as zeros
        for (int i = threadIdx.x; i < kKC * RU; i += 256) b_s[i] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        __syncthreads();
    }
#pragma unroll
    for (int t = 0; t < kPieces; ++t) {
        const int f = t * 256 + (int)threadIdx.x;
        if (f * 4 < total) {
            const float pv[4] = {piece[t].x, piece[t].y, piece[t].z, piece[t].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int idx = f * 4 + e;
                const int kk = idx / N, j = idx - kk * N;
                b_f[((kk & 3) * (kKC / 4) + (kk >> 2)) * (RU * 4) + j] = pv[e];
            }
        }
    }
    __syncthreads();
    float acc[4][NP];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < NP; ++j) acc[r][j] = 0.0f;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const int g4 = u * 32 + lane;
        if (g4 * 4 < kn) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float b[NP];
#pragma unroll
                for (int q = 0; q < NQ; ++q) {
                    const float4 t = b_s[(e * (kKC / 4) + g4) * RU + q];
                    b[q * 4] = t.x; b[q * 4 + 1] = t.y; b[q * 4 + 2] = t.z; b[q * 4 + 3] = t.w;
                }
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    const float av = e == 0 ? a[u][r].x : e == 1 ? a[u][r].y : e == 2 ? a[u][r].z : a[u][r].w;
#pragma unroll
                    for (int j = 0; j < NP; ++j) acc[r][j] = fmaf(av, b[j], acc[r][j]);
                }
            }
        }
    }
    // the 32 lanes' partial sums of a row meet in shared memory; lane j adds column j over the lanes
    float* out = partial + (int64_t)blockIdx.y * M * N;
    __syncthreads();                              // every warp is done with the rows of B: their memory is reused
    float* rs = b_f + warp * 32 * (NP + 1);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        __syncwarp();
#pragma unroll
        for (int j = 0; j < NP; ++j) rs[lane * (NP + 1) + j] = acc[r][j];
        __syncwarp();
        if (lane < N && m0 + r < M) {
            float s = 0.0f;
#pragma unroll 8
            for (int l = 0; l < 32; ++l) s += rs[l * (NP + 1) + lane];
            out[(int64_t)(m0 + r) * N + lane] = s;
        }
    }
    // ---- the block that finishes last for this group of 32 rows folds the k slices, in ascending order
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(&tickets[blockIdx.x], 1) == (int)gridDim.y - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int nsplit = gridDim.y;
    for (int idx = threadIdx.x; idx < 32 * N; idx += 256) {
        const int row = idx / N, col = idx - row * N;
        const int m = blockIdx.x * 32 + row;
        if (m >= M) continue;
        float s = 0.0f;
        for (int sp = 0; sp < nsplit; ++sp) s += __ldcg(partial + ((int64_t)sp * M + m) * N + col);
        if (bias) s += __ldg(bias + col);         // ADD.forward after DOT.forward
        float* c = C + (int64_t)m * N + col;
        *c = accumulate ? *c + s : s;
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
    for (int idx = threadIdx.x; idx < kn * p.N; idx += 256) {   // consecutive threads, consecutive floats
        const int64_t off = (int64_t)kg * 256 * p.N + idx;
        float s = 0.0f;
        for (int q = 0; q < p.msplit; ++q) s += __ldcg(p.partial + (int64_t)q * p.K * p.N + off);
        p.dB[off] = p.acc_db ? p.dB[off] + s : s;
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
    // k extent per block: enough blocks (two fit an SM) to fill the machine
    const int rb = (int)((M + 31) / 32);
    int kc = kKC;
    while (kc > 128 && (int64_t)rb * ((K + kc - 1) / kc) < 2ll * ctx->sm_count) kc >>= 1;
    const int nsplit = (int)((K + kc - 1) / kc);
    void* ws;
    int32_t rc = mtl_workspace(ctx, (size_t)nsplit * M * N * 4, &ws);
    if (rc) return rc;
    dim3 grid((unsigned)rb, (unsigned)nsplit);
    MTL_REQUIRE(ctx, nsplit <= 65535, "Linear: reduction too long");
#define MTL_LIN_FWD(NQ_) mtl_launch_pdl(ctx, k_linear_fwd<NQ_>, grid, dim3(256), (size_t)0, C, (float*)ws, ctx->tickets, A, B, bias, \
                                        (int)M, (int)N, (int)K, kc, 0)
    if (N <= 4) MTL_LIN_FWD(1);
    else if (N <= 8) MTL_LIN_FWD(2);
    else if (N <= 12) MTL_LIN_FWD(3);
    else MTL_LIN_FWD(4);
#undef MTL_LIN_FWD
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
