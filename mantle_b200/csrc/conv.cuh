// Geometry and internal entry points shared by the CONV2D translation units.
#pragma once

#include "common.cuh"

struct ConvGeom {
    int N, C, H, W;  // input
    int K, R, S;     // kernel [K, C, R, S]
    int OH, OW;      // output spatial extent
    int ph, pw, sh, sw, dh, dw;
};

int32_t mtl_sum_partials(mtl_ctx* ctx, float* out, const float* partial, int64_t n, int nsplit, int accumulate);

// CUDA-core kernels (conv_simt.cu)
// relu != 0: Y = relu(conv + bias), applied in the kernel's epilogue where the kernel has one and by an
// in-place pass otherwise
int32_t mtl_conv_fwd_simt(mtl_ctx* ctx, float* Y, const float* X, const float* Wt, const float* bias,
                          const ConvGeom& g, int relu);
int32_t mtl_conv_dgrad_simt(mtl_ctx* ctx, float* dX, const float* ug, const float* Wt, const ConvGeom& g,
                            int accumulate);
int32_t mtl_conv_wgrad_simt(mtl_ctx* ctx, float* dW, const float* ug, const float* X, const ConvGeom& g,
                            int accumulate);
int32_t mtl_conv_bgrad(mtl_ctx* ctx, float* db, const float* ug, const ConvGeom& g, int accumulate);

// First-layer kernel that also pools (conv_simt.cu).
bool mtl_conv_fwd_pool_simt_supported(const ConvGeom& g, const float* pooled);
int32_t mtl_conv_fwd_pool_simt(mtl_ctx* ctx, float* pooled, int32_t* idx, float* pooled_cl, const float* X,
                               const float* Wt, const float* bias, const ConvGeom& g, int relu);

// Kernel and bias gradient of a first layer from the POOLED upper gradient (conv_simt.cu).
bool mtl_conv_wgrad_rows_pooled_supported(const ConvGeom& g);
int32_t mtl_conv_wgrad_bias_rows_pooled(mtl_ctx* ctx, float* dW, float* db, const float* pg, const int32_t* pidx,
                                        const float* pv, const float* X, const ConvGeom& g, int relu, int acc_dw,
                                        int acc_db);

// Tensor-core implicit-GEMM kernels (conv_tc.cu); *_supported says whether a geometry qualifies.
bool mtl_conv_fwd_tc_supported(const ConvGeom& g, const float* X, const float* Wt, const float* Y);
bool mtl_conv_dgrad_tc_supported(const ConvGeom& g, const float* ug, const float* Wt, const float* dX);
bool mtl_conv_wgrad_tc_supported(const ConvGeom& g, const float* ug, const float* X, const float* dW);
// X_cl (may be null): a channels-last copy of X the caller already holds; used in plain TF32 mode.
int32_t mtl_conv_fwd_tc(mtl_ctx* ctx, float* Y, const float* X, const float* Wt, const float* bias,
                        const ConvGeom& g, int x3, int relu, const float* X_cl);
int32_t mtl_channels_last_copy(mtl_ctx* ctx, float* dst, const float* src, int N, int C, int HW);
// First layer (C*R*S <= 32) with RELU and 2x2 pooling on the tensor cores, plain TF32 mode.
bool mtl_conv_first_pool_tc_supported(const ConvGeom& g, const float* X, const float* pooled, const int32_t* idx);
int32_t mtl_conv_first_pool_tc(mtl_ctx* ctx, float* pooled, int32_t* idx, float* pooled_cl, const float* X,
                               const float* Wt, const float* bias, const ConvGeom& g, int relu);
bool mtl_conv_first_wgrad_tc_supported(const ConvGeom& g, const float* X, const float* pg, const int32_t* pidx,
                                       const float* pv);
int32_t mtl_conv_first_wgrad_tc(mtl_ctx* ctx, float* dW, float* db, const float* pg, const int32_t* pidx,
                                const float* pv, const float* X, const ConvGeom& g, int relu, int acc_dw, int acc_db);
bool mtl_conv_fwd_pool_tc_supported(const ConvGeom& g, const float* X, const float* Wt, const float* pooled);
int32_t mtl_conv_fwd_pool_tc(mtl_ctx* ctx, float* pooled, int32_t* idx, const float* X, const float* Wt,
                             const float* bias, const ConvGeom& g, int x3, int relu, const float* X_cl);
int32_t mtl_conv_dgrad_tc(mtl_ctx* ctx, float* dX, const float* ug, const float* Wt, const ConvGeom& g,
                          int accumulate, int x3);
int32_t mtl_conv_wgrad_tc(mtl_ctx* ctx, float* dW, const float* ug, const float* X, const ConvGeom& g,
                          int accumulate, int x3);
// dX, dW and optionally db (may be null) from one channels-last copy of ug.
int32_t mtl_conv_bwd_fused_tc(mtl_ctx* ctx, float* dX, float* dW, float* db, const float* ug, const float* X,
                              const float* Wt, const ConvGeom& g, int acc_dx, int acc_dw, int acc_db, int x3,
                              const float* X_cl);
int32_t mtl_conv_bwd_fused_tc_src(mtl_ctx* ctx, float* dX, float* dW, float* db, const float* ug, const float* pg,
                                  const int32_t* pidx, const float* pv, int relu, const float* X, const float* Wt,
                                  const ConvGeom& g, int acc_dx, int acc_dw, int acc_db, int x3, const float* X_cl);
// Row-streaming first-layer kernel: dW and db in one pass over ug; false when the geometry does not qualify.
bool mtl_conv_wgrad_rows_supported(const ConvGeom& g, const float* ug);
int32_t mtl_conv_wgrad_bias_rows(mtl_ctx* ctx, float* dW, float* db, const float* ug, const float* X, const ConvGeom& g,
                                 int acc_dw, int acc_db);
