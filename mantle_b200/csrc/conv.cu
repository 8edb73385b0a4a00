// CONV2D entry points: argument checks and the choice between the tensor-core implicit-GEMM
// kernels and the CUDA-core kernels.
#include "conv.cuh"

namespace {

int32_t make_geom(mtl_ctx* ctx, const mtl_conv2d_desc* d, ConvGeom* g) {
    MTL_REQUIRE(ctx, d, "null descriptor");
    MTL_REQUIRE(ctx, d->K >= 1, "CONV2D needs at least one output channel");
    int32_t OH, OW;
    if (mtl_conv2d_out_shape(d, &OH, &OW) != MTL_OK)
        return mtl_set_error(ctx, MTL_ERR_INVALID, "convolution geometry gives an empty or invalid output");
    g->N = d->N; g->C = d->C; g->H = d->H; g->W = d->W; g->K = d->K; g->R = d->R; g->S = d->S;
    g->OH = OH; g->OW = OW;
    g->ph = d->pad[0]; g->pw = d->pad[1]; g->sh = d->stride[0]; g->sw = d->stride[1];
    g->dh = d->dilation[0]; g->dw = d->dilation[1];
    return MTL_OK;
}

}  // namespace

extern "C" {

static int32_t conv2d_fwd(mtl_ctx* ctx, float* Y, const float* X, const float* Wt, const float* bias,
                          const mtl_conv2d_desc* d, int relu, const float* X_cl = nullptr) {
    MTL_CHECK_CTX(ctx);
    ConvGeom g;
    int32_t rc = make_geom(ctx, d, &g);
    if (rc) return rc;
    MTL_REQUIRE(ctx, Y && X && Wt, "null pointer in CONV2D forward");
    if (ctx->math_mode != MTL_MATH_FP32 && mtl_conv_fwd_tc_supported(g, X, Wt, Y))
        return mtl_conv_fwd_tc(ctx, Y, X, Wt, bias, g, ctx->math_mode == MTL_MATH_TF32X3, relu, X_cl);
    return mtl_conv_fwd_simt(ctx, Y, X, Wt, bias, g, relu);
}

int32_t mtl_conv2d_fwd(mtl_ctx* ctx, float* Y, const float* X, const float* Wt, const float* bias,
                       const mtl_conv2d_desc* d) {
    return conv2d_fwd(ctx, Y, X, Wt, bias, d, 0);
}

int32_t mtl_conv2d_fwd_act(mtl_ctx* ctx, float* Y, const float* X, const float* Wt, const float* bias,
                           const mtl_conv2d_desc* d, int32_t act_op) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, act_op == MTL_OP_RELU || act_op < 0, "mtl_conv2d_fwd_act fuses RELU only (act_op %d)", act_op);
    return conv2d_fwd(ctx, Y, X, Wt, bias, d, act_op == MTL_OP_RELU ? 1 : 0);
}

int32_t mtl_conv2d_bwd(mtl_ctx* ctx, int32_t tensor_id, float* grad, const float* ug, const float* X,
                       const float* Wt, const mtl_conv2d_desc* d, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    ConvGeom g;
    int32_t rc = make_geom(ctx, d, &g);
    if (rc) return rc;
    MTL_REQUIRE(ctx, tensor_id >= 0 && tensor_id <= 2, "tensor_id must be 0, 1 or 2");
    MTL_REQUIRE(ctx, grad && ug, "null pointer in mtl_conv2d_bwd");
    const bool tc = ctx->math_mode != MTL_MATH_FP32;
    const int x3 = ctx->math_mode == MTL_MATH_TF32X3;
    if (tensor_id == 0) {
        MTL_REQUIRE(ctx, Wt, "input gradient needs the kernel");
        if (tc && mtl_conv_dgrad_tc_supported(g, ug, Wt, grad))
            return mtl_conv_dgrad_tc(ctx, grad, ug, Wt, g, accumulate, x3);
        return mtl_conv_dgrad_simt(ctx, grad, ug, Wt, g, accumulate);
    }
    if (tensor_id == 1) {
        MTL_REQUIRE(ctx, X, "kernel gradient needs the input");
        if (tc && mtl_conv_wgrad_tc_supported(g, ug, X, grad))
            return mtl_conv_wgrad_tc(ctx, grad, ug, X, g, accumulate, x3);
        return mtl_conv_wgrad_simt(ctx, grad, ug, X, g, accumulate);
    }
    return mtl_conv_bgrad(ctx, grad, ug, g, accumulate);
}

int32_t mtl_conv2d_fwd_act_pool(mtl_ctx* ctx, float* pooled, int32_t* idx, const float* X, const float* Wt,
                                const float* bias, const mtl_conv2d_desc* d, int32_t act_op,
                                const mtl_conv2d_desc* pool) {
    return mtl_conv2d_fwd_act_pool_cl(ctx, pooled, idx, nullptr, X, nullptr, Wt, bias, d, act_op, pool);
}

int32_t mtl_conv2d_fwd_act_pool_cl(mtl_ctx* ctx, float* pooled, int32_t* idx, float* pooled_cl, const float* X,
                                   const float* X_cl, const float* Wt, const float* bias, const mtl_conv2d_desc* d,
                                   int32_t act_op, const mtl_conv2d_desc* pool) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, act_op == MTL_OP_RELU || act_op < 0, "mtl_conv2d_fwd_act_pool fuses RELU only (act_op %d)", act_op);
    ConvGeom g;
    int32_t rc = make_geom(ctx, d, &g);
    if (rc) return rc;
    MTL_REQUIRE(ctx, pooled && X && Wt && pool, "null pointer in mtl_conv2d_fwd_act_pool");
    MTL_REQUIRE(ctx, pool->N == g.N && pool->C == g.K && pool->H == g.OH && pool->W == g.OW,
                "the pooling descriptor does not describe the convolution's output");
    const int relu = act_op == MTL_OP_RELU ? 1 : 0;
    const bool pool_2x2 = pool->R == 2 && pool->S == 2 && pool->stride[0] == 2 && pool->stride[1] == 2 &&
                          pool->pad[0] == 0 && pool->pad[1] == 0 && pool->dilation[0] == 1 && pool->dilation[1] == 1 &&
                          g.OH % 2 == 0 && g.OW % 2 == 0;
    const bool tc = ctx->math_mode != MTL_MATH_FP32 && mtl_conv_fwd_tc_supported(g, X, Wt, pooled);
    if (pool_2x2 && !tc && ctx->math_mode == MTL_MATH_TF32 && mtl_conv_first_pool_tc_supported(g, X, pooled, idx))
        return mtl_conv_first_pool_tc(ctx, pooled, idx, pooled_cl, X, Wt, bias, g, relu);
    if (pool_2x2 && !tc && mtl_conv_fwd_pool_simt_supported(g, pooled))
        return mtl_conv_fwd_pool_simt(ctx, pooled, idx, pooled_cl, X, Wt, bias, g, relu);
    if (pool_2x2 && tc && mtl_conv_fwd_pool_tc_supported(g, X, Wt, pooled)) {
        // the implicit-GEMM kernel pools in its epilogue: the activation never reaches memory
        rc = mtl_conv_fwd_pool_tc(ctx, pooled, idx, X, Wt, bias, g, ctx->math_mode == MTL_MATH_TF32X3, relu, X_cl);
        if (rc || !pooled_cl) return rc;
        return mtl_channels_last_copy(ctx, pooled_cl, pooled, g.N, g.K, (g.OH / 2) * (g.OW / 2));
    }
    // no kernel pools this geometry in its epilogue: the activation goes through scratch memory
    void* scratch;
    rc = mtl_workspace2(ctx, (size_t)g.N * g.K * g.OH * g.OW * 4, &scratch);
    if (rc) return rc;
    rc = conv2d_fwd(ctx, (float*)scratch, X, Wt, bias, d, relu, X_cl);
    if (rc) return rc;
    rc = mtl_maxpool2d_fwd(ctx, pooled, idx, (const float*)scratch, pool);
    if (rc || !pooled_cl) return rc;
    int32_t POH, POW;
    if (mtl_conv2d_out_shape(pool, &POH, &POW) != MTL_OK) return mtl_set_error(ctx, MTL_ERR_INVALID, "bad pooling geometry");
    return mtl_channels_last_copy(ctx, pooled_cl, pooled, g.N, g.K, POH * POW);
}

int32_t mtl_conv2d_bwd_pooled(mtl_ctx* ctx, float* dX, float* dW, float* db, const float* pooled_ug,
                              const int32_t* idx, const float* pooled, const float* X, const float* X_cl,
                              const float* Wt, const mtl_conv2d_desc* d, int32_t act_op, const mtl_conv2d_desc* pool,
                              int32_t acc_dx, int32_t acc_dw, int32_t acc_db) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, act_op == MTL_OP_RELU || act_op < 0, "mtl_conv2d_bwd_pooled fuses RELU only (act_op %d)", act_op);
    ConvGeom g;
    int32_t rc = make_geom(ctx, d, &g);
    if (rc) return rc;
    MTL_REQUIRE(ctx, pooled_ug && idx && pool && (dX || dW || db), "null pointer in mtl_conv2d_bwd_pooled");
    MTL_REQUIRE(ctx, (!dX || Wt) && (!dW || X), "operand needed by a requested gradient is null");
    MTL_REQUIRE(ctx, act_op < 0 || pooled, "the fused RELU gradient needs the pooled output");
    MTL_REQUIRE(ctx, pool->N == g.N && pool->C == g.K && pool->H == g.OH && pool->W == g.OW,
                "the pooling descriptor does not describe the convolution's output");
    const int relu = act_op == MTL_OP_RELU ? 1 : 0;
    const bool pool_2x2 = pool->R == 2 && pool->S == 2 && pool->stride[0] == 2 && pool->stride[1] == 2 &&
                          pool->pad[0] == 0 && pool->pad[1] == 0 && pool->dilation[0] == 1 && pool->dilation[1] == 1 &&
                          g.OH % 2 == 0 && g.OW % 2 == 0;
    const bool tc_mode = ctx->math_mode != MTL_MATH_FP32;
    const int x3 = ctx->math_mode == MTL_MATH_TF32X3;
    // tensor-core layer: the pooled gradient is scattered straight into the channels-last operand copy
    if (pool_2x2 && tc_mode && dX && dW && mtl_conv_dgrad_tc_supported(g, pooled_ug, Wt, dX) &&
        mtl_conv_wgrad_tc_supported(g, pooled_ug, X, dW) && (size_t)(g.OH / 2) * (g.OW / 2) <= 784)
        return mtl_conv_bwd_fused_tc_src(ctx, dX, dW, db, nullptr, pooled_ug, idx, pooled, relu, X, Wt, g, acc_dx, acc_dw,
                                         acc_db, x3, X_cl);
    // first layer on CUDA cores: the dense gradient is rebuilt in shared memory
    const bool wgrad_tc = tc_mode && dW && mtl_conv_wgrad_tc_supported(g, pooled_ug, X, dW);
    if (pool_2x2 && !dX && !wgrad_tc && ctx->math_mode == MTL_MATH_TF32 && (dW || db) &&
        mtl_conv_first_wgrad_tc_supported(g, X, pooled_ug, idx, relu ? pooled : pooled_ug))
        return mtl_conv_first_wgrad_tc(ctx, dW, db, pooled_ug, idx, pooled, X, g, relu, acc_dw, acc_db);
    if (pool_2x2 && !dX && !wgrad_tc && mtl_conv_wgrad_rows_pooled_supported(g))
        return mtl_conv_wgrad_bias_rows_pooled(ctx, dW, db, pooled_ug, idx, pooled, X, g, relu, acc_dw, acc_db);
    // no kernel consumes the pooled form for this geometry: the dense gradient passes through scratch
    void* scratch;
    rc = mtl_workspace2(ctx, (size_t)g.N * g.K * g.OH * g.OW * 4, &scratch);
    if (rc) return rc;
    rc = mtl_maxpool2d_bwd_idx_act(ctx, (float*)scratch, pooled_ug, idx, pooled, pool, relu ? MTL_OP_RELU : -1, 0);
    if (rc) return rc;
    return mtl_conv2d_bwd_fused_cl(ctx, dX, dW, db, (const float*)scratch, X, X_cl, Wt, d, acc_dx, acc_dw, acc_db);
}

int32_t mtl_conv2d_bwd_fused(mtl_ctx* ctx, float* dX, float* dW, float* db, const float* ug, const float* X,
                             const float* Wt, const mtl_conv2d_desc* d, int32_t acc_dx, int32_t acc_dw, int32_t acc_db) {
    return mtl_conv2d_bwd_fused_cl(ctx, dX, dW, db, ug, X, nullptr, Wt, d, acc_dx, acc_dw, acc_db);
}

int32_t mtl_conv2d_bwd_fused_cl(mtl_ctx* ctx, float* dX, float* dW, float* db, const float* ug, const float* X,
                                const float* X_cl, const float* Wt, const mtl_conv2d_desc* d, int32_t acc_dx,
                                int32_t acc_dw, int32_t acc_db) {
    MTL_CHECK_CTX(ctx);
    ConvGeom g;
    int32_t rc = make_geom(ctx, d, &g);
    if (rc) return rc;
    MTL_REQUIRE(ctx, ug && (dX || dW || db), "null pointer in mtl_conv2d_bwd_fused");
    MTL_REQUIRE(ctx, (!dX || Wt) && (!dW || X), "operand needed by a requested gradient is null");
    const bool tc = ctx->math_mode != MTL_MATH_FP32;
    const int x3 = ctx->math_mode == MTL_MATH_TF32X3;
    if (tc && dX && dW && mtl_conv_dgrad_tc_supported(g, ug, Wt, dX) && mtl_conv_wgrad_tc_supported(g, ug, X, dW))
        return mtl_conv_bwd_fused_tc(ctx, dX, dW, db, ug, X, Wt, g, acc_dx, acc_dw, acc_db, x3, X_cl);
    if (dW && db && !(tc && mtl_conv_wgrad_tc_supported(g, ug, X, dW)) && mtl_conv_wgrad_rows_supported(g, ug)) {
        rc = mtl_conv_wgrad_bias_rows(ctx, dW, db, ug, X, g, acc_dw, acc_db);
        if (rc) return rc;
        dW = nullptr;
        db = nullptr;
    }
    // whatever is left: one reference-shaped call per operand
    if (dX && (rc = mtl_conv2d_bwd(ctx, 0, dX, ug, X, Wt, d, acc_dx))) return rc;
    if (dW && (rc = mtl_conv2d_bwd(ctx, 1, dW, ug, X, Wt, d, acc_dw))) return rc;
    if (db && (rc = mtl_conv2d_bwd(ctx, 2, db, ug, X, Wt, d, acc_db))) return rc;
    return MTL_OK;
}

}  // extern "C"
