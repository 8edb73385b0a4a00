/*
 * mantle_oracle.c -- CPU restatement of Mantle's operator kernels and Adam step.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA backend is compared against (and
 * the timed CPU baseline); nothing in the shipped library or the mantle_b200 package calls it.
 *
 * The reference is written in Mojo (toolchain mojo 1.0.0b3.dev2026061606, pixi.toml:22) and cannot
 * be executed where this is built, so every function below restates one reference function in
 * plain C, keeping its loop order and arithmetic wherever they determine the result.  Each
 * function cites the reference lines it follows.  Pinning: tests/test_oracle_kat.py checks these
 * functions against the known-answer values in the reference's own tests (the .mojo files under tests/mojo) and
 * against fixtures generated with PyTorch CPU, which is the oracle the reference's tests/python/ files
 * use (tests/golden/make_golden.py).
 *
 * Where the reference's result depends on the host SIMD width (`nelts = 2 * simd_width`,
 * mantle/__init__.mojo:21) the lane count is fixed to MO_NELTS = 16 (the AVX2 value); such sums
 * are compared with a tolerance, never bit-for-bit.
 *
 * Threading follows the reference's `parallelize` call sites through OpenMP: dot over row blocks
 * (matmul.mojo:133), conv forward / input gradient over the batch (conv.mojo:171,224,338), kernel
 * and bias gradient over output channels (conv.mojo:393,423), axis reductions over outputs
 * (tensorutils.mojo:682).  Pooling and broadcast paths are serial as in the reference.
 *
 * Build: see oracle/Makefile (gcc -O3 -march=x86-64-v3 -ffp-contract=off -fopenmp -shared).
 */
#ifdef _OPENMP
#include <omp.h>
#endif
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MO_NELTS 16
#define MO_MAX_RANK 8
#define MO_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------ helpers ------------- */

static int64_t mo_numel(int rank, const int64_t* shape) {
    int64_t n = 1;
    for (int i = 0; i < rank; ++i) n *= shape[i];
    return n;
}

/* Host threads the parallel loops below use.  The reference forks one task per row block / image /
 * channel on all host cores (std.algorithm.parallelize); launchers such as torch.distributed.run
 * export OMP_NUM_THREADS=1 for multi-process jobs, so a timing harness sets the count explicitly. */
MO_API void mo_set_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
MO_API int mo_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* broadcast_shapes, mantle/core/tensorutils.mojo:89-127. Returns rank, or -1 if incompatible. */
MO_API int mo_broadcast_shapes(int r1, const int64_t* s1, int r2, const int64_t* s2, int64_t* out) {
    int ndim = r1 > r2 ? r1 : r2;
    int diff = r1 > r2 ? r1 - r2 : r2 - r1;
    const int64_t* big = r1 > r2 ? s1 : s2;
    const int64_t* small = r1 > r2 ? s2 : s1;
    for (int i = ndim - 1; i >= diff; --i) {
        int64_t a = big[i], b = small[i - diff];
        if (a == b) out[i] = a;
        else if (a == 1 || b == 1) out[i] = a * b;
        else return -1;
    }
    for (int i = diff - 1; i >= 0; --i) out[i] = big[i];
    return ndim;
}

/* broadcast_calculate_strides, tensorutils.mojo:150-175 */
static void mo_bcast_strides(int size, int rank, const int64_t* shape, int64_t* strides) {
    int diff = size - rank;
    for (int i = 0; i < size; ++i) strides[i] = 0;
    int64_t stride = 1;
    for (int i = rank - 1; i >= 0; --i) {
        if (shape[i] != 1) {
            strides[i + diff] = stride;
            stride *= shape[i];
        }
    }
}

/* get_real_index, tensorutils.mojo:51-82 */
static int64_t mo_real_index(int size, const int64_t* strides, const int64_t* bshape, int64_t i) {
    int64_t res = 0, lin = i;
    for (int j = size - 1; j >= 0; --j) {
        res += (lin % bshape[j]) * strides[j];
        lin /= bshape[j];
    }
    return res;
}

static int mo_is_scalar(int rank, const int64_t* shape) { return rank == 1 && shape[0] == 1; }
static int mo_same_shape(int r1, const int64_t* s1, int r2, const int64_t* s2) {
    if (r1 != r2) return 0;
    for (int i = 0; i < r1; ++i)
        if (s1[i] != s2[i]) return 0;
    return 1;
}

/* fill, tensorutils.mojo:30-44 */
MO_API void mo_fill(float* t, int64_t n, float v) {
    for (int64_t i = 0; i < n; ++i) t[i] = v;
}

/* ------------------------------------------------------------------ matmul -------------- */

/* dot + calculate_block, mantle/autograd/ops/matmul.mojo:26-153: res[M,N] = t1[M,K] . t2[K,N].
 * Every output element is acc = fma(t1[m,k], t2[k,n], acc) for k ascending (:50-62); the 6x16
 * tiling only decides which elements a thread owns, so the result does not depend on it. */
MO_API void mo_dot(float* res, const float* t1, const float* t2, int64_t M, int64_t K, int64_t N) {
    enum { BM = 6, BN = 16 };
    int64_t mblocks = (M + BM - 1) / BM;
#pragma omp parallel for schedule(static)
    for (int64_t mb = 0; mb < mblocks; ++mb) {
        int64_t m0 = mb * BM;
        int64_t mh = M - m0 < BM ? M - m0 : BM;
        for (int64_t n0 = 0; n0 < N; n0 += BN) {
            int64_t nw = N - n0 < BN ? N - n0 : BN;
            float acc[BM][BN];
            memset(acc, 0, sizeof(acc));
            for (int64_t k = 0; k < K; ++k) {
                const float* brow = t2 + k * N + n0;
                for (int64_t m = 0; m < mh; ++m) {
                    float a = t1[(m0 + m) * K + k];
                    for (int64_t n = 0; n < nw; ++n) acc[m][n] = fmaf(a, brow[n], acc[m][n]);
                }
            }
            for (int64_t m = 0; m < mh; ++m)
                for (int64_t n = 0; n < nw; ++n) res[(m0 + m) * N + n0 + n] = acc[m][n];
        }
    }
}

/* transpose_2D, tensorutils.mojo:494-522 */
static float* mo_transpose_2d(const float* t, int64_t rows, int64_t cols) {
    float* out = (float*)malloc(sizeof(float) * (size_t)(rows * cols));
    for (int64_t i = 0; i < rows; ++i)
        for (int64_t j = 0; j < cols; ++j) out[j * rows + i] = t[i * cols + j];
    return out;
}

/* dot_transpose_t2, matmul.mojo:175-182: res[M,K] = ug[M,N] . t2[K,N]^T */
MO_API void mo_dot_transpose_t2(float* res, const float* ug, const float* t2, int64_t M, int64_t K, int64_t N) {
    float* t2t = mo_transpose_2d(t2, K, N); /* [N, K] */
    mo_dot(res, ug, t2t, M, N, K);
    free(t2t);
}

/* dot_transpose_t1, matmul.mojo:203-210: res[K,N] = t1[M,K]^T . ug[M,N] */
MO_API void mo_dot_transpose_t1(float* res, const float* t1, const float* ug, int64_t M, int64_t K, int64_t N) {
    float* t1t = mo_transpose_2d(t1, M, K); /* [K, M] */
    mo_dot(res, t1t, ug, K, M, N);
    free(t1t);
}

/* ------------------------------------------------------------------ conv / pool --------- */

typedef struct {
    int32_t N, C, H, W;
    int32_t K, R, S;
    int32_t pad[2], stride[2], dilation[2];
} mo_conv_desc;

/* get_result_shape, mantle/autograd/ops/conv.mojo:25-58 (floor division as Mojo's //) */
static int64_t mo_floordiv(int64_t a, int64_t b) {
    int64_t q = a / b;
    if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
    return q;
}
MO_API void mo_conv_out_shape(const mo_conv_desc* d, int32_t* OH, int32_t* OW) {
    *OH = (int32_t)(mo_floordiv((int64_t)d->H + 2 * d->pad[0] - (int64_t)d->dilation[0] * (d->R - 1) - 1, d->stride[0]) + 1);
    *OW = (int32_t)(mo_floordiv((int64_t)d->W + 2 * d->pad[1] - (int64_t)d->dilation[1] * (d->S - 1) - 1, d->stride[1]) + 1);
}

/* CONV2D.forward, conv.mojo:81-226: zero-filled im2col buffer [batch, oX*oY, C*kX*kY], then one
 * dot product per output in MO_NELTS-lane partial sums + horizontal add + bias (:178-222). */
MO_API void mo_conv2d_fwd(float* out, const float* in, const float* kernel, const float* bias, const mo_conv_desc* d) {
    int32_t OH, OW;
    mo_conv_out_shape(d, &OH, &OW);
    const int64_t crs = (int64_t)d->C * d->R * d->S;
    const int64_t col_batch = (int64_t)OH * OW * crs;
    float* col = (float*)calloc((size_t)(d->N * col_batch), sizeof(float));
#pragma omp parallel for schedule(static)
    for (int b = 0; b < d->N; ++b)
        for (int ux = 0; ux < OH; ++ux)
            for (int uy = 0; uy < OW; ++uy)
                for (int c = 0; c < d->C; ++c)
                    for (int kx = 0; kx < d->R; ++kx)
                        for (int ky = 0; ky < d->S; ++ky) {
                            int ix = ux * d->stride[0] - d->pad[0] + kx * d->dilation[0];
                            int iy = uy * d->stride[1] - d->pad[1] + ky * d->dilation[1];
                            if (ix < 0 || iy < 0 || ix >= d->H || iy >= d->W) continue;
                            col[b * col_batch + ((int64_t)ux * OW + uy) * crs + ((int64_t)c * d->R * d->S + kx * d->S + ky)] =
                                in[(((int64_t)b * d->C + c) * d->H + ix) * d->W + iy];
                        }
#pragma omp parallel for schedule(static)
    for (int b = 0; b < d->N; ++b)
        for (int k = 0; k < d->K; ++k)
            for (int ux = 0; ux < OH; ++ux)
                for (int uy = 0; uy < OW; ++uy) {
                    float lanes[MO_NELTS];
                    for (int l = 0; l < MO_NELTS; ++l) lanes[l] = 0.0f;
                    const float* cp = col + b * col_batch + ((int64_t)ux * OW + uy) * crs;
                    const float* kp = kernel + (int64_t)k * crs;
                    int64_t i = 0;
                    for (; i + MO_NELTS <= crs; i += MO_NELTS)
                        for (int l = 0; l < MO_NELTS; ++l) lanes[l] += cp[i + l] * kp[i + l];
                    for (; i < crs; ++i) lanes[0] += cp[i] * kp[i]; /* width-1 remainder calls */
                    float r = 0.0f;
                    for (int l = 0; l < MO_NELTS; ++l) r += lanes[l];
                    out[(((int64_t)b * d->K + k) * OH + ux) * OW + uy] = r + bias[k];
                }
    free(col);
}

/* CONV2D.backward, conv.mojo:229-425.  `res` is overwritten with the operand's gradient
 * (the caller accumulates, ops.mojo:498). tensor_id 0: input (:284-338), 1: kernel (:340-393),
 * 2: bias (:395-423). */
MO_API void mo_conv2d_bwd(int tensor_id, float* res, const float* ug, const float* in, const float* kernel,
                          const mo_conv_desc* d) {
    int32_t OH, OW;
    mo_conv_out_shape(d, &OH, &OW);
    if (tensor_id == 0) {
        memset(res, 0, sizeof(float) * (size_t)d->N * d->C * d->H * d->W);
#pragma omp parallel for schedule(static)
        for (int b = 0; b < d->N; ++b)
            for (int k = 0; k < d->K; ++k)
                for (int ux = 0; ux < OH; ++ux)
                    for (int uy = 0; uy < OW; ++uy) {
                        int ix_base = ux * d->stride[0] - d->pad[0];
                        int iy_base = uy * d->stride[1] - d->pad[1];
                        float ug_val = ug[(((int64_t)b * d->K + k) * OH + ux) * OW + uy];
                        for (int c = 0; c < d->C; ++c)
                            for (int kx = 0; kx < d->R; ++kx)
                                for (int ky = 0; ky < d->S; ++ky) {
                                    int ix = ix_base + kx * d->dilation[0];
                                    int iy = iy_base + ky * d->dilation[1];
                                    if (ix < 0 || iy < 0 || ix >= d->H || iy >= d->W) continue;
                                    res[(((int64_t)b * d->C + c) * d->H + ix) * d->W + iy] +=
                                        kernel[(((int64_t)k * d->C + c) * d->R + kx) * d->S + ky] * ug_val;
                                }
                    }
    } else if (tensor_id == 1) {
#pragma omp parallel for schedule(static)
        for (int k = 0; k < d->K; ++k)
            for (int64_t q = 0; q < (int64_t)d->C * d->R * d->S; ++q) {
                int c = (int)(q / (d->R * d->S));
                int kx = (int)((q / d->S) % d->R);
                int ky = (int)(q % d->S);
                float result = 0.0f;
                for (int b = 0; b < d->N; ++b)
                    for (int ux = 0; ux < OH; ++ux)
                        for (int uy = 0; uy < OW; ++uy) {
                            int ix = ux * d->stride[0] - d->pad[0] + kx * d->dilation[0];
                            int iy = uy * d->stride[1] - d->pad[1] + ky * d->dilation[1];
                            if (ix < 0 || iy < 0 || ix >= d->H || iy >= d->W) continue;
                            result += in[(((int64_t)b * d->C + c) * d->H + ix) * d->W + iy] *
                                      ug[(((int64_t)b * d->K + k) * OH + ux) * OW + uy];
                        }
                res[(int64_t)k * d->C * d->R * d->S + q] = result;
            }
    } else {
#pragma omp parallel for schedule(static)
        for (int k = 0; k < d->K; ++k) {
            float sum = 0.0f;
            int64_t plane = (int64_t)OH * OW;
            for (int b = 0; b < d->N; ++b) {
                const float* p = ug + ((int64_t)b * d->K + k) * plane;
                int64_t i = 0;
                for (; i + MO_NELTS <= plane; i += MO_NELTS) {
                    float chunk = 0.0f;
                    for (int l = 0; l < MO_NELTS; ++l) chunk += p[i + l];
                    sum += chunk;
                }
                for (; i < plane; ++i) sum += p[i];
            }
            res[k] = sum;
        }
    }
}

/* MAXPOOL2D.forward, mantle/autograd/ops/pool.mojo:44-100.  `idx` (optional) receives the
 * plane-local offset of the selected element, -1 when no element exceeded -inf. */
MO_API void mo_maxpool2d_fwd(float* out, int32_t* idx, const float* in, const mo_conv_desc* d) {
    int32_t OH, OW;
    mo_conv_out_shape(d, &OH, &OW);
    for (int b = 0; b < d->N; ++b)
        for (int c = 0; c < d->C; ++c)
            for (int x = 0; x < OH; ++x)
                for (int y = 0; y < OW; ++y) {
                    float max_val = -INFINITY;
                    int32_t max_idx = -1;
                    int ix_base = x * d->stride[0] - d->pad[0];
                    int iy_base = y * d->stride[1] - d->pad[1];
                    for (int kx = 0; kx < d->R; ++kx)
                        for (int ky = 0; ky < d->S; ++ky) {
                            int ix = ix_base + kx * d->dilation[0];
                            int iy = iy_base + ky * d->dilation[1];
                            if (ix < 0 || iy < 0 || ix >= d->H || iy >= d->W) continue;
                            float val = in[(((int64_t)b * d->C + c) * d->H + ix) * d->W + iy];
                            if (val > max_val) {
                                max_val = val;
                                max_idx = ix * d->W + iy;
                            }
                        }
                    int64_t o = (((int64_t)b * d->C + c) * OH + x) * OW + y;
                    out[o] = max_val;
                    if (idx) idx[o] = max_idx;
                }
}

/* MAXPOOL2D.backward, pool.mojo:103-165.  The reference writes res[-1] when a window selects
 * nothing (:128,163); here such a window contributes nothing. */
MO_API void mo_maxpool2d_bwd(float* res, const float* ug, const float* in, const mo_conv_desc* d) {
    int32_t OH, OW;
    mo_conv_out_shape(d, &OH, &OW);
    memset(res, 0, sizeof(float) * (size_t)d->N * d->C * d->H * d->W);
    for (int b = 0; b < d->N; ++b)
        for (int c = 0; c < d->C; ++c)
            for (int x = 0; x < OH; ++x)
                for (int y = 0; y < OW; ++y) {
                    float max_val = -INFINITY;
                    int64_t max_idx = -1;
                    int ix_base = x * d->stride[0] - d->pad[0];
                    int iy_base = y * d->stride[1] - d->pad[1];
                    for (int kx = 0; kx < d->R; ++kx)
                        for (int ky = 0; ky < d->S; ++ky) {
                            int ix = ix_base + kx * d->dilation[0];
                            int iy = iy_base + ky * d->dilation[1];
                            if (ix < 0 || iy < 0 || ix >= d->H || iy >= d->W) continue;
                            int64_t i = (((int64_t)b * d->C + c) * d->H + ix) * d->W + iy;
                            if (in[i] > max_val) {
                                max_val = in[i];
                                max_idx = i;
                            }
                        }
                    if (max_idx >= 0) res[max_idx] += ug[(((int64_t)b * d->C + c) * OH + x) * OW + y];
                }
}

/* ------------------------------------------------------------------ elementwise --------- */

enum {
    MO_ADD = 0, MO_SUB = 1, MO_MUL = 2, MO_DIV = 3, MO_EXP = 4, MO_LOG = 5, MO_POW = 6,
    MO_SUM = 8, MO_MEAN = 9, MO_MAX = 10, MO_SIGMOID = 13, MO_RELU = 14, MO_TANH = 15,
    MO_CLIP = 20, MO_LEAKYRELU = 28
};

static float mo_bin(int op, float a, float b) {
    switch (op) {
        case MO_ADD: return a + b;
        case MO_SUB: return a - b;
        case MO_MUL: return a * b;
        default: return a / b;
    }
}

/* elwise_op dispatch + broadcast_elwise_op, tensorutils.mojo:243-357 */
MO_API int mo_binary_fwd(int op, float* res, const float* t1, const float* t2, int r1, const int64_t* s1, int r2,
                         const int64_t* s2) {
    int64_t bs[MO_MAX_RANK];
    int rank = mo_broadcast_shapes(r1, s1, r2, s2, bs);
    if (rank < 0) return -1;
    int64_t n = mo_numel(rank, bs);
    if (mo_is_scalar(r2, s2)) {
        for (int64_t i = 0; i < n; ++i) res[i] = mo_bin(op, t1[i], t2[0]);
    } else if (mo_is_scalar(r1, s1)) {
        for (int64_t i = 0; i < n; ++i) res[i] = mo_bin(op, t1[0], t2[i]);
    } else if (!mo_same_shape(r1, s1, r2, s2)) {
        int64_t st1[MO_MAX_RANK], st2[MO_MAX_RANK];
        mo_bcast_strides(rank, r1, s1, st1);
        mo_bcast_strides(rank, r2, s2, st2);
        for (int64_t i = 0; i < n; ++i)
            res[i] = mo_bin(op, t1[mo_real_index(rank, st1, bs, i)], t2[mo_real_index(rank, st2, bs, i)]);
    } else {
        for (int64_t i = 0; i < n; ++i) res[i] = mo_bin(op, t1[i], t2[i]);
    }
    return 0;
}

/* ADD/SUB/MUL/DIV.backward (basics.mojo:46-219) followed by the un-broadcasting accumulate_grad
 * of backward_op (ops.mojo:457-463, tensorutils.mojo:455-487): grad += d(out)/d(operand). */
MO_API int mo_binary_bwd(int op, int tensor_id, float* grad, const float* ug, const float* t1, const float* t2,
                         int r1, const int64_t* s1, int r2, const int64_t* s2) {
    int64_t bs[MO_MAX_RANK];
    int rank = mo_broadcast_shapes(r1, s1, r2, s2, bs);
    if (rank < 0) return -1;
    int64_t n = mo_numel(rank, bs);
    float* rg = (float*)malloc(sizeof(float) * (size_t)n);
    int64_t st1[MO_MAX_RANK], st2[MO_MAX_RANK];
    mo_bcast_strides(rank, r1, s1, st1);
    mo_bcast_strides(rank, r2, s2, st2);
    int b_scalar = mo_is_scalar(r2, s2);
    for (int64_t i = 0; i < n; ++i) {
        float a = t1 ? t1[mo_real_index(rank, st1, bs, i)] : 0.0f;
        float b = t2 ? t2[mo_real_index(rank, st2, bs, i)] : 0.0f;
        float u = ug[i], v;
        switch (op) {
            case MO_ADD: v = u; break;
            case MO_SUB: v = tensor_id == 0 ? u : u * -1.0f; break;
            case MO_MUL: v = tensor_id == 0 ? u * b : u * a; break;
            default:
                if (tensor_id == 0) v = u / b;
                else if (b_scalar) v = (-1.0f / (b * b)) * a * u; /* basics.mojo:168-178 */
                else v = -a / (b * b) * u;                         /* basics.mojo:191-215 */
        }
        rg[i] = v;
    }
    int gr = tensor_id == 0 ? r1 : r2;
    const int64_t* gs = tensor_id == 0 ? s1 : s2;
    if (mo_same_shape(gr, gs, rank, bs)) {
        for (int64_t i = 0; i < n; ++i) grad[i] += rg[i];
    } else if (mo_is_scalar(rank, bs)) {
        int64_t ng = mo_numel(gr, gs);
        for (int64_t i = 0; i < ng; ++i) grad[i] += rg[0];
    } else {
        int64_t stg[MO_MAX_RANK];
        mo_bcast_strides(rank, gr, gs, stg);
        for (int64_t i = 0; i < n; ++i) grad[mo_real_index(rank, stg, bs, i)] += rg[i];
    }
    free(rg);
    return 0;
}

static float mo_powi(float x, int n) {
    int neg = n < 0;
    unsigned e = neg ? (unsigned)(-(long long)n) : (unsigned)n;
    float r = 1.0f, b = x;
    while (e) {
        if (e & 1u) r *= b;
        b *= b;
        e >>= 1;
    }
    return neg ? 1.0f / r : r;
}

/* elwise_transform / elwise_pow users: EXP, LOG (basics.mojo:260-309), POW (:312-327),
 * SIGMOID, RELU, LEAKYRELU, TANH, CLIP (mlops.mojo:27-299). */
MO_API void mo_unary_fwd(int op, float* res, const float* t, int64_t n, float p0, float p1) {
    for (int64_t i = 0; i < n; ++i) {
        float x = t[i], y;
        switch (op) {
            case MO_EXP: y = expf(x); break;
            case MO_LOG: y = logf(x); break;
            case MO_POW: y = mo_powi(x, (int)p0); break;
            case MO_SIGMOID: y = 1.0f / (1.0f + expf(-x)); break;
            case MO_RELU: y = x > 0.0f ? x : 0.0f; break;
            case MO_TANH: y = (expf(x) - expf(-x)) / (expf(x) + expf(-x)); break;
            case MO_CLIP: y = fmaxf(fminf(x, p1), p0); break;
            case MO_LEAKYRELU: y = x > 0.0f ? x : x * p0; break;
            default: y = x;
        }
        res[i] = y;
    }
}

/* The matching backward arms; grad += local_gradient(t) * ug (ops.mojo:405). */
MO_API void mo_unary_bwd(int op, float* grad, const float* ug, const float* t, int64_t n, float p0, float p1) {
    for (int64_t i = 0; i < n; ++i) {
        float x = t[i], u = ug[i], v;
        switch (op) {
            case MO_EXP: v = expf(x) * u; break;
            case MO_LOG: v = u / x; break;
            case MO_POW: v = p0 * powf(x + 1e-12f, p0 - 1.0f) * u; break; /* basics.mojo:350-355 */
            case MO_SIGMOID: {
                float s = 1.0f / (1.0f + expf(-x));
                v = s * (1.0f - s) * u;
                break;
            }
            case MO_RELU: v = (x > 0.0f ? 1.0f : 0.0f) * u; break;
            case MO_TANH: {
                float th = (expf(x) - expf(-x)) / (expf(x) + expf(-x));
                v = (1.0f - th * th) * u;
                break;
            }
            case MO_CLIP: v = (x >= p0 && x <= p1) ? u : 0.0f; break;
            case MO_LEAKYRELU: v = (x > 0.0f ? 1.0f : p0) * u; break;
            default: v = u;
        }
        grad[i] += v;
    }
}

/* POW.backward for the exponent (basics.mojo:359-376): grad[0] += sum_i x_i^a * log(x_i) * ug_i with
 * log(x) replaced by 0 where it is infinite (x == 0); the reference sums nelts-lane partial sums
 * (host dependent), here the running fp32 sum in index order -- tolerance-compared. */
MO_API void mo_pow_bwd_exponent(float* grad, const float* ug, const float* t, int64_t n, float a) {
    float acc = grad[0];
    for (int64_t i = 0; i < n; ++i) {
        float lg = logf(t[i]);
        if (isinf(lg)) lg = 0.0f;
        acc += powf(t[i], a) * lg * ug[i];
    }
    grad[0] = acc;
}

/* ------------------------------------------------------------------ reductions ---------- */

/* reduce (whole tensor), tensorutils.mojo:565-598: MO_NELTS running lanes, width-1 tail into
 * lane 0, horizontal fold. */
static float mo_reduce_all(const float* t, int64_t n, int is_max) {
    float lanes[MO_NELTS];
    for (int l = 0; l < MO_NELTS; ++l) lanes[l] = is_max ? -FLT_MAX : 0.0f;
    int64_t i = 0;
    for (; i + MO_NELTS <= n; i += MO_NELTS)
        for (int l = 0; l < MO_NELTS; ++l) lanes[l] = is_max ? fmaxf(lanes[l], t[i + l]) : lanes[l] + t[i + l];
    for (; i < n; ++i) lanes[0] = is_max ? fmaxf(lanes[0], t[i]) : lanes[0] + t[i];
    float r = lanes[0];
    for (int l = 1; l < MO_NELTS; ++l) r = is_max ? fmaxf(r, lanes[l]) : r + lanes[l];
    return r;
}

/* reduce (axis), tensorutils.mojo:623-684 */
static void mo_reduce_axis(float* res, const float* t, int rank, const int64_t* shape, int axis, int is_max) {
    int64_t n = mo_numel(rank, shape), dim = shape[axis], stride = 1;
    for (int d = axis + 1; d < rank; ++d) stride *= shape[d];
    int64_t n_out = n / dim;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n_out; ++i) {
        float lanes[MO_NELTS];
        for (int l = 0; l < MO_NELTS; ++l) lanes[l] = is_max ? -FLT_MAX : 0.0f;
        int64_t base = (i % stride) + (i / stride) * (stride * dim);
        int64_t j = 0;
        for (; j + MO_NELTS <= dim; j += MO_NELTS)
            for (int l = 0; l < MO_NELTS; ++l) {
                float v = t[base + (j + l) * stride];
                lanes[l] = is_max ? fmaxf(lanes[l], v) : lanes[l] + v;
            }
        for (; j < dim; ++j) {
            float v = t[base + j * stride];
            lanes[0] = is_max ? fmaxf(lanes[0], v) : lanes[0] + v;
        }
        float r = lanes[0];
        for (int l = 1; l < MO_NELTS; ++l) r = is_max ? fmaxf(r, lanes[l]) : r + lanes[l];
        res[i] = r;
    }
}

/* SUM/MEAN/MAX.forward, basics.mojo:393-406, 441-452, 522-534; tmean :710-720, :761-772 */
MO_API void mo_reduce_fwd(int op, float* res, const float* t, int rank, const int64_t* shape, int axis) {
    int64_t n = mo_numel(rank, shape);
    if (axis < 0) {
        float r = mo_reduce_all(t, n, op == MO_MAX);
        res[0] = op == MO_MEAN ? r / (float)n : r;
        return;
    }
    mo_reduce_axis(res, t, rank, shape, axis, op == MO_MAX);
    if (op == MO_MEAN) {
        int64_t n_out = n / shape[axis];
        float dimf = (float)shape[axis];
        for (int64_t i = 0; i < n_out; ++i) res[i] = res[i] / dimf;
    }
}

/* SUM/MEAN/MAX.backward, basics.mojo:409-425, 455-506, 537-615; grad += result (ops.mojo:405).
 * accumulate_op applies its function a second time when both shapes are equal
 * (tensorutils.mojo:380-393); that is kept. */
MO_API void mo_reduce_bwd(int op, float* grad, const float* ug, const float* t, int rank, const int64_t* shape,
                          int axis) {
    int64_t n = mo_numel(rank, shape);
    int64_t dim = axis >= 0 ? shape[axis] : n, stride = 1;
    for (int d = axis + 1; axis >= 0 && d < rank; ++d) stride *= shape[d];
    if (op == MO_SUM || op == MO_MEAN) {
        float coef = 1.0f;
        int twice = 0;
        if (op == MO_SUM) twice = axis >= 0 ? dim == 1 : (rank == 1 && shape[0] == 1);
        else if (axis < 0) coef = (float)(1.0 / (double)n);
        else { coef = (float)(1.0 / (double)dim); twice = dim == 1; }
        for (int64_t i = 0; i < n; ++i) {
            int64_t u = axis < 0 ? 0 : (i % stride) + (i / (stride * dim)) * stride;
            float r = coef * ug[u];
            if (twice) r = r * ug[u];
            grad[i] += r;
        }
        return;
    }
    if (axis < 0) {
        float mx = mo_reduce_all(t, n, 1);
        float cnt = 0.0f;
        for (int64_t i = 0; i < n; ++i)
            if (t[i] == mx) cnt += 1.0f;
        float factor = 1.0f / cnt;
        for (int64_t i = 0; i < n; ++i)
            if (t[i] == mx) grad[i] += factor * ug[0];
        return;
    }
    int64_t n_out = n / dim;
    float* mxs = (float*)malloc(sizeof(float) * (size_t)n_out);
    mo_reduce_axis(mxs, t, rank, shape, axis, 1);
    for (int64_t i = 0; i < n_out; ++i) {
        int64_t base = (i % stride) + (i / stride) * (stride * dim);
        float cnt = 0.0f;
        for (int64_t j = 0; j < dim; ++j)
            if (t[base + j * stride] == mxs[i]) cnt += 1.0f;
        float factor = 1.0f / cnt;
        for (int64_t j = 0; j < dim; ++j)
            if (t[base + j * stride] == mxs[i]) grad[base + j * stride] += factor * ug[i];
    }
    free(mxs);
}

/* ------------------------------------------------------------------ Adam ---------------- */

static float mo_pow_int(float b, int e) {
    float r = 1.0f;
    while (e > 0) {
        if (e & 1) r *= b;
        b *= b;
        e >>= 1;
    }
    return r;
}

/* Adam.step for one parameter tensor, mantle/nn/optim.mojo:104-138. `iter` is the count after the
 * increment at :96.  grads are scaled by grad_scale first (1 for the reference's single process). */
MO_API void mo_adam_step(float* params, const float* grads, float* m, float* v, int64_t n, float lr, float beta1,
                         float beta2, float eps, int iter, float grad_scale) {
    float c1 = 1.0f - mo_pow_int(beta1, iter);
    float c2 = 1.0f - mo_pow_int(beta2, iter);
    float omb1 = 1.0f - beta1, omb2 = 1.0f - beta2;
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < n; ++j) {
        float g = grads[j] * grad_scale;
        float mm = beta1 * m[j] + omb1 * g;
        m[j] = mm;
        mm = mm / c1;
        float vv = beta2 * v[j] + omb2 * g * g;
        v[j] = vv;
        vv = vv / c2;
        params[j] = params[j] - lr * (mm / (sqrtf(vv) + eps));
    }
}

MO_API int mo_nelts(void) { return MO_NELTS; }
