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

}  // namespace

int32_t mtl_gemm_simt(mtl_ctx* ctx, float* C, const float* A, const float* B, int64_t M, int64_t N, int64_t K,
                      int transA, int transB, int accumulate) {
    MTL_REQUIRE(ctx, M >= 1 && N >= 1 && K >= 1 && M < (1ll << 31) && N < (1ll << 31) && K < (1ll << 31),
                "DOT extents out of range (M=%lld K=%lld N=%lld)", (long long)M, (long long)K, (long long)N);
    if (N <= 16) {
        dim3 grid((unsigned)((N + 15) / 16), (unsigned)((M + 255) / 256));
        MTL_REQUIRE(ctx, grid.y <= 65535u, "DOT: M too large for the skinny kernel");
        k_gemm_simt<256, 16, 16, 4, 4><<<grid, 256, 0, ctx->stream>>>(C, A, B, (int)M, (int)N, (int)K, transA, transB, accumulate);
    } else {
        dim3 grid((unsigned)((N + 63) / 64), (unsigned)((M + 63) / 64));
        MTL_REQUIRE(ctx, grid.y <= 65535u, "DOT: M too large for the CUDA-core kernel");
        k_gemm_simt<64, 64, 16, 4, 4><<<grid, 256, 0, ctx->stream>>>(C, A, B, (int)M, (int)N, (int)K, transA, transB, accumulate);
    }
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}
