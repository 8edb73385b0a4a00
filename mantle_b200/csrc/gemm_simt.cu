// CUDA-core fp32 GEMM for OP.DOT: the exact mode and the path for shapes the tensor-core kernel
// cannot take (row strides that are not multiples of 16 bytes, tiny extents).
// Every output element is one fmaf chain over k = 0..K-1 in ascending order, which is the
// accumulation order of calculate_block (mantle/autograd/ops/matmul.mojo:50-62), so results are
// bit-identical to the reference's dot for any tiling chosen here.
#include "common.cuh"

namespace {

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
k_gemm_simt(float* __restrict__ C, const float* __restrict__ A, const float* __restrict__ B, int M, int N, int K,
            int transA, int transB, int accumulate) {
    mtl_pdl_sync();
    constexpr int NT = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN);  // column group
    const int ty = tid / (BN / TN);  // row group
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        // stage A tile: element (m, k)
        for (int e = tid; e < BM * BK; e += NT) {
            int mm, kk;
            if (transA) { mm = e % BM; kk = e / BM; }   // A stored [K, M]: m contiguous
            else        { kk = e % BK; mm = e / BK; }   // A stored [M, K]: k contiguous
            int m = m0 + mm, k = k0 + kk;
            float v = 0.0f;
            if (m < M && k < K) v = transA ? A[(int64_t)k * M + m] : A[(int64_t)m * K + k];
            As[kk][mm] = v;
        }
        for (int e = tid; e < BN * BK; e += NT) {
            int nn, kk;
            if (transB) { kk = e % BK; nn = e / BK; }   // B stored [N, K]: k contiguous
            else        { nn = e % BN; kk = e / BN; }   // B stored [K, N]: n contiguous
            int n = n0 + nn, k = k0 + kk;
            float v = 0.0f;
            if (n < N && k < K) v = transB ? B[(int64_t)n * K + k] : B[(int64_t)k * N + n];
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            int n = n0 + tx * TN + j;
            if (n >= N) continue;
            int64_t o = (int64_t)m * N + n;
            C[o] = accumulate ? C[o] + acc[i][j] : acc[i][j];
        }
    }
}

// ---- thin products (N <= 16), e.g. the classifier of the CNNs: [B, 6272] . [6272, 10] -------------
// These are bound by reading A once.  They re-associate the k sum (lane / split partials), so they
// are used only outside MTL_MATH_FP32; results differ from the ascending chain by fp32 rounding.

// C[M,N] = A[M,K] . B[K,N], A row-major: one warp per ROWS rows, lanes stride over k.
template <int ROWS>
__global__ void __launch_bounds__(128) k_gemm_thin_n(float* __restrict__ C, const float* __restrict__ A,
                                                     const float* __restrict__ B, int M, int N, int K,
                                                     int accumulate) {
    mtl_pdl_sync();
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    const int m0 = warp * ROWS;
    if (m0 >= M) return;
    float acc[ROWS][16];
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int j = 0; j < 16; ++j) acc[r][j] = 0.0f;
    for (int k = lane; k < K; k += 32) {
        float b[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) b[j] = j < N ? __ldg(B + (int64_t)k * N + j) : 0.0f;
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            float a = (m0 + r < M) ? __ldg(A + (int64_t)(m0 + r) * K + k) : 0.0f;
#pragma unroll
            for (int j = 0; j < 16; ++j) acc[r][j] = fmaf(a, b[j], acc[r][j]);
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            float v = acc[r][j];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && j < N && m0 + r < M) {
                int64_t idx = (int64_t)(m0 + r) * N + j;
                C[idx] = accumulate ? C[idx] + v : v;
            }
        }
}

// partial[split][M,N] = A[M, k-slice] . B[k-slice, N]: a block stages its slice of B in shared
// memory (rows padded to 20 floats so that the four float4 reads of a row are conflict free), each
// warp streams four rows of A with coalesced loads and keeps 4 x 16 partial sums per lane.
// Splitting k gives enough blocks to fill the machine when M is only a few thousand rows.
constexpr int kThinKC = 512;  // k extent of one block
// NQ: float4 groups of a row of B that are multiplied (N rounded up to a multiple of four columns).
template <int NQ>
__global__ void __launch_bounds__(256, 3) k_gemm_thin_tile(float* __restrict__ partial, const float* __restrict__ A,
                                                        const float* __restrict__ B, int M, int N, int K) {
    mtl_pdl_sync();
    constexpr int NP = 4 * NQ;
    __shared__ __align__(16) float b_s[kThinKC * 20];
    const int k_begin = blockIdx.y * kThinKC;
    const int kn = min(kThinKC, K - k_begin);
    for (int i = threadIdx.x; i < kn * 16; i += 256) {
        const int kk = i >> 4, j = i & 15;
        b_s[kk * 20 + j] = j < N ? __ldg(B + (int64_t)(k_begin + kk) * N + j) : 0.0f;
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = (blockIdx.x * 8 + warp) * 4;   // rows past M load zeros and store nothing
    float acc[4][NP];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < NP; ++j) acc[r][j] = 0.0f;
    const float* a0 = A + (int64_t)m0 * K + k_begin;
    // four k steps at a time: their sixteen loads of A are in flight together (the kernel is bound by
    // the latency of streaming A, not by arithmetic)
    for (int kk0 = lane; kk0 < kn; kk0 += 128) {
        float a[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int r = 0; r < 4; ++r)
                a[u][r] = (kk0 + 32 * u < kn && m0 + r < M) ? __ldg(a0 + (int64_t)r * K + kk0 + 32 * u) : 0.0f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int kk = kk0 + 32 * u;
            if (kk < kn) {
                float b[NP];
#pragma unroll
                for (int q = 0; q < NQ; ++q) {
                    const float4 t = *reinterpret_cast<const float4*>(b_s + kk * 20 + q * 4);
                    b[q * 4] = t.x; b[q * 4 + 1] = t.y; b[q * 4 + 2] = t.z; b[q * 4 + 3] = t.w;
                }
#pragma unroll
                for (int r = 0; r < 4; ++r)
#pragma unroll
                    for (int j = 0; j < NP; ++j) acc[r][j] = fmaf(a[u][r], b[j], acc[r][j]);
            }
        }
    }
    // the 32 lanes' partial sums of a row meet in shared memory: lane j then adds column j over the lanes
    // in ascending order (cheaper than a five-step shuffle tree per value)
    float* out = partial + (int64_t)blockIdx.y * M * N;
    __syncthreads();                              // every warp is done with the rows of B: their memory is reused
    float* rs = b_s + warp * 32 * (NP + 1);       // per warp: the lanes' partial sums of one row, odd row stride
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
}

// partial[split][M,N] = A^T . B over a slice of k, A stored [K, M] (m contiguous): one thread per
// output row, rows of B staged in shared memory.
template <int NQ>
__global__ void __launch_bounds__(256) k_gemm_thin_n_ta(float* __restrict__ partial, const float* __restrict__ A,
                                                        const float* __restrict__ B, int M, int N, int K,
                                                        int k_per_split) {
    mtl_pdl_sync();
    constexpr int NP = 4 * NQ;   // N rounded up to whole float4 groups
    __shared__ __align__(16) float b_s[64][16];
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    const int k_begin = blockIdx.y * k_per_split;
    const int k_end = min(K, k_begin + k_per_split);
    float acc[NP];
#pragma unroll
    for (int j = 0; j < NP; ++j) acc[j] = 0.0f;
    for (int k0 = k_begin; k0 < k_end; k0 += 64) {
        __syncthreads();
        for (int i = threadIdx.x; i < 64 * 16; i += blockDim.x) {
            int kk = i >> 4, j = i & 15;
            b_s[kk][j] = (k0 + kk < k_end && j < N) ? __ldg(B + (int64_t)(k0 + kk) * N + j) : 0.0f;
        }
        __syncthreads();
        if (m < M) {
            const int kn = min(64, k_end - k0);
            for (int kk0 = 0; kk0 < kn; kk0 += 8) {   // eight loads of A in flight
                float a[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) a[u] = kk0 + u < kn ? __ldg(A + (int64_t)(k0 + kk0 + u) * M + m) : 0.0f;
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (kk0 + u < kn) {
#pragma unroll
                        for (int q = 0; q < NQ; ++q) {
                            const float4 t = *reinterpret_cast<const float4*>(&b_s[kk0 + u][4 * q]);
                            acc[4 * q] = fmaf(a[u], t.x, acc[4 * q]);
                            acc[4 * q + 1] = fmaf(a[u], t.y, acc[4 * q + 1]);
                            acc[4 * q + 2] = fmaf(a[u], t.z, acc[4 * q + 2]);
                            acc[4 * q + 3] = fmaf(a[u], t.w, acc[4 * q + 3]);
                        }
                    }
                }
            }
        }
    }
    if (m < M) {
        float* out = partial + ((int64_t)blockIdx.y * M + m) * N;
#pragma unroll
        for (int j = 0; j < NP; ++j)       // static indices: the accumulators stay in registers
            if (j < N) out[j] = acc[j];
    }
}

__global__ void __launch_bounds__(256) k_fold_partials(float* __restrict__ out, const float* __restrict__ partial,
                                                       int64_t n, int nsplit, int accumulate) {
    mtl_pdl_sync();
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) {
        float s = 0.0f;
        int j = 0;
        for (; j + 8 <= nsplit; j += 8) {   // eight partials in flight, added in ascending order
            float t[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) t[u] = partial[(int64_t)(j + u) * n + i];
#pragma unroll
            for (int u = 0; u < 8; ++u) s += t[u];
        }
        for (; j < nsplit; ++j) s += partial[(int64_t)j * n + i];
        out[i] = accumulate ? out[i] + s : s;
    }
}

}  // namespace

bool mtl_gemm_thin_supported(int64_t M, int64_t N, int64_t K, int transA, int transB) {
    return N <= 16 && !transB && M * K >= (1 << 16) && M < (1ll << 31) && K < (1ll << 31);
}

int32_t mtl_gemm_thin(mtl_ctx* ctx, float* C, const float* A, const float* B, int64_t M, int64_t N, int64_t K,
                      int transA, int accumulate) {
    if (!transA && K >= 2 * kThinKC) {
        const int nsplit = (int)((K + kThinKC - 1) / kThinKC);
        void* ws;
        int32_t rc = mtl_workspace(ctx, (size_t)nsplit * M * N * 4, &ws);
        if (rc) return rc;
        dim3 grid((unsigned)((M + 31) / 32), (unsigned)nsplit);
        if (N <= 4) mtl_launch_pdl(ctx, k_gemm_thin_tile<1>, dim3(grid), dim3(256), (size_t)(0), (float*)ws, A, B, (int)M, (int)N, (int)K);
        else if (N <= 8) mtl_launch_pdl(ctx, k_gemm_thin_tile<2>, dim3(grid), dim3(256), (size_t)(0), (float*)ws, A, B, (int)M, (int)N, (int)K);
        else if (N <= 12) mtl_launch_pdl(ctx, k_gemm_thin_tile<3>, dim3(grid), dim3(256), (size_t)(0), (float*)ws, A, B, (int)M, (int)N, (int)K);
        else mtl_launch_pdl(ctx, k_gemm_thin_tile<4>, dim3(grid), dim3(256), (size_t)(0), (float*)ws, A, B, (int)M, (int)N, (int)K);
        MTL_LAUNCHED(ctx);
        int fg = mtl_grid_for(M * N, 256, ctx->sm_count, 8);
        mtl_launch_pdl(ctx, k_fold_partials, dim3(fg), dim3(256), (size_t)(0), C, (const float*)ws, M * N, nsplit, accumulate);
        MTL_LAUNCHED(ctx);
        return MTL_OK;
    }
    if (!transA) {
        constexpr int ROWS = 4;
        int64_t warps = (M + ROWS - 1) / ROWS;
        int grid = (int)((warps * 32 + 127) / 128);
        mtl_launch_pdl(ctx, k_gemm_thin_n<ROWS>, dim3(grid), dim3(128), (size_t)(0), C, A, B, (int)M, (int)N, (int)K, accumulate);
        MTL_LAUNCHED(ctx);
        return MTL_OK;
    }
    int gx = (int)((M + 255) / 256);
    int nsplit = (ctx->sm_count * 4 + gx - 1) / gx;
    int64_t kps = (K + nsplit - 1) / nsplit;
    kps = (kps + 63) / 64 * 64;
    nsplit = (int)((K + kps - 1) / kps);
    void* ws;
    int32_t rc = mtl_workspace(ctx, (size_t)nsplit * M * N * 4, &ws);
    if (rc) return rc;
    dim3 grid((unsigned)gx, (unsigned)nsplit);
    if (N <= 4) mtl_launch_pdl(ctx, k_gemm_thin_n_ta<1>, dim3(grid), dim3(256), (size_t)(0), (float*)ws, A, B, (int)M, (int)N, (int)K, (int)kps);
    else if (N <= 8) mtl_launch_pdl(ctx, k_gemm_thin_n_ta<2>, dim3(grid), dim3(256), (size_t)(0), (float*)ws, A, B, (int)M, (int)N, (int)K, (int)kps);
    else if (N <= 12) mtl_launch_pdl(ctx, k_gemm_thin_n_ta<3>, dim3(grid), dim3(256), (size_t)(0), (float*)ws, A, B, (int)M, (int)N, (int)K, (int)kps);
    else mtl_launch_pdl(ctx, k_gemm_thin_n_ta<4>, dim3(grid), dim3(256), (size_t)(0), (float*)ws, A, B, (int)M, (int)N, (int)K, (int)kps);
    MTL_LAUNCHED(ctx);
    int fg = mtl_grid_for(M * N, 256, ctx->sm_count, 8);
    mtl_launch_pdl(ctx, k_fold_partials, dim3(fg), dim3(256), (size_t)(0), C, (const float*)ws, M * N, nsplit, accumulate);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

int32_t mtl_gemm_simt(mtl_ctx* ctx, float* C, const float* A, const float* B, int64_t M, int64_t N, int64_t K,
                      int transA, int transB, int accumulate) {
    MTL_REQUIRE(ctx, M >= 1 && N >= 1 && K >= 1 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31),
                "DOT extents out of range (M=%lld K=%lld N=%lld)", (long long)M, (long long)K, (long long)N);
    if (N <= 16) {
        dim3 grid((unsigned)((N + 15) / 16), (unsigned)((M + 255) / 256));
        MTL_REQUIRE(ctx, grid.y <= 65535u, "DOT: M too large for the skinny kernel");
        mtl_launch_pdl(ctx, k_gemm_simt<256, 16, 16, 4, 4>, dim3(grid), dim3(256), (size_t)(0), C, A, B, (int)M, (int)N, (int)K, transA, transB, accumulate);
    } else {
        dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64));
        MTL_REQUIRE(ctx, grid.y <= 65535u, "DOT: M too large for the CUDA-core kernel");
        mtl_launch_pdl(ctx, k_gemm_simt<64, 64, 16, 4, 4>, dim3(grid), dim3(256), (size_t)(0), C, A, B, (int)M, (int)N, (int)K, transA, transB, accumulate);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}
