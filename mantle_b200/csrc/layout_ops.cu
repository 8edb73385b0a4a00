// TRANSPOSE, SLICE, CONCAT and SPLIT, forward and backward: all are strided copies.  One kernel
// walks a region (rank <= 8) and moves dst[doff + i . dstride] (+)= src[soff + i . sstride]; the entry
// points only differ in how they set the region, the strides and the offsets.  HBM-bound; the
// contiguous side of every copy is coalesced, the permuted side of a TRANSPOSE is not tiled.
#include "common.cuh"

namespace {

constexpr int kBlock = 256;

struct Region {
    int rank;
    int narrow;  // every extent and offset fits 32 bits
    int64_t shape[MTL_MAX_RANK];
    int64_t ds[MTL_MAX_RANK], ss[MTL_MAX_RANK];
    int64_t doff, soff;
};

__global__ void __launch_bounds__(kBlock) k_strided_copy(float* __restrict__ dst, const float* __restrict__ src, int64_t n,
                                                         Region r, int acc) {
    int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = tid; i < n; i += stride) {
        int64_t d = r.doff, s = r.soff;
        if (r.narrow) {
            uint32_t j = (uint32_t)i;
#pragma unroll
            for (int a = MTL_MAX_RANK - 1; a >= 0; --a) {
                if (a < r.rank) {
                    const uint32_t e = (uint32_t)r.shape[a];
                    const uint32_t q = j / e, m = j - q * e;
                    d += (int64_t)m * r.ds[a];
                    s += (int64_t)m * r.ss[a];
                    j = q;
                }
            }
        } else {
            int64_t j = i;
#pragma unroll
            for (int a = MTL_MAX_RANK - 1; a >= 0; --a) {
                if (a < r.rank) {
                    const int64_t q = j / r.shape[a], m = j - q * r.shape[a];
                    d += m * r.ds[a];
                    s += m * r.ss[a];
                    j = q;
                }
            }
        }
        dst[d] = acc ? dst[d] + src[s] : src[s];
    }
}

void contiguous_strides(int rank, const int64_t* shape, int64_t* st) {
    int64_t s = 1;
    for (int d = rank - 1; d >= 0; --d) { st[d] = s; s *= shape[d]; }
}

int32_t run_copy(mtl_ctx* ctx, float* dst, const float* src, Region& r, int acc) {
    int64_t n = 1;
    for (int d = 0; d < r.rank; ++d) n *= r.shape[d];
    if (n == 0) return MTL_OK;
    r.narrow = n < (1ll << 31) ? 1 : 0;
    for (int d = r.rank; d < MTL_MAX_RANK; ++d) { r.shape[d] = 1; r.ds[d] = 0; r.ss[d] = 0; }
    int grid = mtl_grid_for(n, kBlock, ctx->sm_count, 8);
    k_strided_copy<<<grid, kBlock, 0, ctx->stream>>>(dst, src, n, r, acc);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

bool shape_ok(int32_t rank, const int64_t* shape) {
    if (rank < 1 || rank > MTL_MAX_RANK || !shape) return false;
    for (int i = 0; i < rank; ++i)
        if (shape[i] < 1) return false;
    return true;
}

// TRANSPOSE.result_shape / forward (basics.mojo:618-662): axes == null reverses the axes.
bool make_perm(int32_t rank, const int32_t* axes, int* perm) {
    bool seen[MTL_MAX_RANK] = {false};
    for (int i = 0; i < rank; ++i) {
        int a = axes ? axes[i] : rank - 1 - i;
        if (a < 0 || a >= rank || seen[a]) return false;
        seen[a] = true;
        perm[i] = a;
    }
    return true;
}

// SLICE.adjust_boundary (mlops.mojo:378-382)
int64_t adjust_boundary(int64_t s, int64_t dim) {
    int64_t v = s >= 0 ? s : dim + s;
    return v > dim ? dim : (v < 0 ? 0 : v);
}
int64_t range_len(int64_t start, int64_t end, int64_t step) {
    if (step > 0) return start < end ? (end - start + step - 1) / step : 0;
    return start > end ? (start - end - step - 1) / (-step) : 0;
}

// reorder_positions (mlops.mojo:456-478): per-axis start and step, and the extent of the result.
int32_t slice_plan(mtl_ctx* ctx, int32_t rank, const int64_t* in_shape, const mtl_slice_desc* d, int64_t* start,
                   int64_t* step, int64_t* out_shape) {
    if (!d || d->n < 0 || d->n > rank) return mtl_set_error(ctx, MTL_ERR_INVALID, "bad slice descriptor");
    for (int a = 0; a < rank; ++a) { start[a] = 0; step[a] = 1; out_shape[a] = in_shape[a]; }
    for (int i = 0; i < d->n; ++i) {
        const int a = d->axes[i] < 0 ? i : d->axes[i];
        if (a >= rank) return mtl_set_error(ctx, MTL_ERR_INVALID, "slice axis %d out of range", a);
        if (d->steps[i] == 0) return mtl_set_error(ctx, MTL_ERR_INVALID, "slice step 0");
        const int64_t s = adjust_boundary(d->starts[i], in_shape[a]), e = adjust_boundary(d->ends[i], in_shape[a]);
        const int64_t len = range_len(s, e, d->steps[i]);
        if (len < 1) return mtl_set_error(ctx, MTL_ERR_INVALID, "slice of axis %d is empty", a);
        // the reference indexes start + i * step without a check; an index outside the axis is refused here
        const int64_t last = s + (len - 1) * d->steps[i];
        if (s >= in_shape[a] || last < 0 || last >= in_shape[a])
            return mtl_set_error(ctx, MTL_ERR_INVALID, "slice of axis %d reaches outside the tensor", a);
        start[a] = s;
        step[a] = d->steps[i];
        out_shape[a] = len;
    }
    return MTL_OK;
}

}  // namespace

extern "C" {

int32_t mtl_transpose_fwd(mtl_ctx* ctx, float* out, const float* in, int32_t rank, const int64_t* in_shape,
                          const int32_t* axes) {
    MTL_CHECK_CTX(ctx);
    int perm[MTL_MAX_RANK];
    MTL_REQUIRE(ctx, out && in && shape_ok(rank, in_shape) && make_perm(rank, axes, perm), "bad arguments to mtl_transpose_fwd");
    int64_t ist[MTL_MAX_RANK];
    contiguous_strides(rank, in_shape, ist);
    Region r;
    r.rank = rank; r.doff = 0; r.soff = 0;
    for (int d = 0; d < rank; ++d) r.shape[d] = in_shape[perm[d]];
    contiguous_strides(rank, r.shape, r.ds);
    for (int d = 0; d < rank; ++d) r.ss[d] = ist[perm[d]];
    return run_copy(ctx, out, in, r, 0);
}

// TRANSPOSE.backward (basics.mojo:664-703): the inverse permutation of ug, added to grad.
int32_t mtl_transpose_bwd(mtl_ctx* ctx, float* grad, const float* ug, int32_t rank, const int64_t* in_shape,
                          const int32_t* axes, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    int perm[MTL_MAX_RANK];
    MTL_REQUIRE(ctx, grad && ug && shape_ok(rank, in_shape) && make_perm(rank, axes, perm), "bad arguments to mtl_transpose_bwd");
    int64_t ist[MTL_MAX_RANK];
    contiguous_strides(rank, in_shape, ist);
    Region r;
    r.rank = rank; r.doff = 0; r.soff = 0;
    for (int d = 0; d < rank; ++d) r.shape[d] = in_shape[perm[d]];   // the region is ug's shape
    contiguous_strides(rank, r.shape, r.ss);
    for (int d = 0; d < rank; ++d) r.ds[d] = ist[perm[d]];
    return run_copy(ctx, grad, ug, r, accumulate ? 1 : 0);
}

int32_t mtl_slice_out_shape(int32_t rank, const int64_t* in_shape, const mtl_slice_desc* d, int64_t* out_shape) {
    if (!shape_ok(rank, in_shape) || !out_shape) return MTL_ERR_INVALID;
    int64_t start[MTL_MAX_RANK], step[MTL_MAX_RANK];
    return slice_plan(nullptr, rank, in_shape, d, start, step, out_shape);
}

int32_t mtl_slice_fwd(mtl_ctx* ctx, float* out, const float* in, int32_t rank, const int64_t* in_shape,
                      const mtl_slice_desc* d) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, out && in && shape_ok(rank, in_shape), "bad arguments to mtl_slice_fwd");
    int64_t start[MTL_MAX_RANK], step[MTL_MAX_RANK], ist[MTL_MAX_RANK];
    Region r;
    int32_t rc = slice_plan(ctx, rank, in_shape, d, start, step, r.shape);
    if (rc) return rc;
    contiguous_strides(rank, in_shape, ist);
    r.rank = rank; r.doff = 0; r.soff = 0;
    contiguous_strides(rank, r.shape, r.ds);
    for (int a = 0; a < rank; ++a) { r.ss[a] = ist[a] * step[a]; r.soff += start[a] * ist[a]; }
    return run_copy(ctx, out, in, r, 0);
}

// SLICE.backward (mlops.mojo:630-656): ug lands on the sliced positions of a zero tensor, which is
// then added to grad.
int32_t mtl_slice_bwd(mtl_ctx* ctx, float* grad, const float* ug, int32_t rank, const int64_t* in_shape,
                      const mtl_slice_desc* d, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, grad && ug && shape_ok(rank, in_shape), "bad arguments to mtl_slice_bwd");
    int64_t start[MTL_MAX_RANK], step[MTL_MAX_RANK], ist[MTL_MAX_RANK];
    Region r;
    int32_t rc = slice_plan(ctx, rank, in_shape, d, start, step, r.shape);
    if (rc) return rc;
    contiguous_strides(rank, in_shape, ist);
    r.rank = rank; r.doff = 0; r.soff = 0;
    contiguous_strides(rank, r.shape, r.ss);
    for (int a = 0; a < rank; ++a) { r.ds[a] = ist[a] * step[a]; r.doff += start[a] * ist[a]; }
    if (!accumulate) MTL_CUDA(ctx, cudaMemsetAsync(grad, 0, (size_t)mtl_numel(rank, in_shape) * 4, ctx->stream));
    return run_copy(ctx, grad, ug, r, accumulate ? 1 : 0);
}

// CONCAT.forward (dynamics.mojo:51-76): inputs agree on every axis except `dim`.
int32_t mtl_concat_fwd(mtl_ctx* ctx, float* out, const float* const* ins, int32_t n_in, int32_t rank,
                       const int64_t* in_shapes, int32_t dim) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, out && ins && in_shapes && n_in >= 1 && rank >= 1 && rank <= MTL_MAX_RANK && dim >= 0 && dim < rank,
                "bad arguments to mtl_concat_fwd");
    int64_t out_shape[MTL_MAX_RANK], ost[MTL_MAX_RANK];
    for (int a = 0; a < rank; ++a) out_shape[a] = in_shapes[a];
    out_shape[dim] = 0;
    for (int j = 0; j < n_in; ++j) {
        const int64_t* s = in_shapes + (int64_t)j * rank;
        MTL_REQUIRE(ctx, shape_ok(rank, s) && ins[j], "bad input %d of mtl_concat_fwd", j);
        for (int a = 0; a < rank; ++a)
            MTL_REQUIRE(ctx, a == dim || s[a] == out_shape[a], "CONCAT inputs differ outside the concatenated axis");
        out_shape[dim] += s[dim];
    }
    contiguous_strides(rank, out_shape, ost);
    int64_t off = 0;
    for (int j = 0; j < n_in; ++j) {
        const int64_t* s = in_shapes + (int64_t)j * rank;
        Region r;
        r.rank = rank; r.soff = 0; r.doff = off * ost[dim];
        for (int a = 0; a < rank; ++a) { r.shape[a] = s[a]; r.ds[a] = ost[a]; }
        contiguous_strides(rank, r.shape, r.ss);
        int32_t rc = run_copy(ctx, out, ins[j], r, 0);
        if (rc) return rc;
        off += s[dim];
    }
    return MTL_OK;
}

// CONCAT.backward (dynamics.mojo:78-108): the slab of ug that input `input_id` produced.
int32_t mtl_concat_bwd(mtl_ctx* ctx, float* grad, const float* ug, int32_t input_id, int32_t n_in, int32_t rank,
                       const int64_t* in_shapes, int32_t dim, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, grad && ug && in_shapes && n_in >= 1 && input_id >= 0 && input_id < n_in && rank >= 1 &&
                         rank <= MTL_MAX_RANK && dim >= 0 && dim < rank, "bad arguments to mtl_concat_bwd");
    int64_t out_shape[MTL_MAX_RANK], ost[MTL_MAX_RANK];
    for (int a = 0; a < rank; ++a) out_shape[a] = in_shapes[a];
    out_shape[dim] = 0;
    int64_t off = 0;
    for (int j = 0; j < n_in; ++j) {
        MTL_REQUIRE(ctx, shape_ok(rank, in_shapes + (int64_t)j * rank), "bad input shape %d", j);
        if (j < input_id) off += in_shapes[(int64_t)j * rank + dim];
        out_shape[dim] += in_shapes[(int64_t)j * rank + dim];
    }
    contiguous_strides(rank, out_shape, ost);
    const int64_t* s = in_shapes + (int64_t)input_id * rank;
    Region r;
    r.rank = rank; r.doff = 0; r.soff = off * ost[dim];
    for (int a = 0; a < rank; ++a) { r.shape[a] = s[a]; r.ss[a] = ost[a]; }
    contiguous_strides(rank, r.shape, r.ds);
    return run_copy(ctx, grad, ug, r, accumulate ? 1 : 0);
}

// SPLIT.forward (dynamics.mojo:138-164): consecutive sections of axis `dim`.
int32_t mtl_split_fwd(mtl_ctx* ctx, float* const* outs, const float* in, int32_t n_out, int32_t rank,
                      const int64_t* in_shape, const int64_t* sections, int32_t dim) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, outs && in && sections && n_out >= 1 && shape_ok(rank, in_shape) && dim >= 0 && dim < rank,
                "bad arguments to mtl_split_fwd");
    int64_t total = 0, ist[MTL_MAX_RANK];
    for (int j = 0; j < n_out; ++j) { MTL_REQUIRE(ctx, sections[j] >= 1 && outs[j], "bad section %d", j); total += sections[j]; }
    MTL_REQUIRE(ctx, total == in_shape[dim], "SPLIT sections sum to %lld, the axis has %lld", (long long)total, (long long)in_shape[dim]);
    contiguous_strides(rank, in_shape, ist);
    int64_t off = 0;
    for (int j = 0; j < n_out; ++j) {
        Region r;
        r.rank = rank; r.doff = 0; r.soff = off * ist[dim];
        for (int a = 0; a < rank; ++a) { r.shape[a] = a == dim ? sections[j] : in_shape[a]; r.ss[a] = ist[a]; }
        contiguous_strides(rank, r.shape, r.ds);
        int32_t rc = run_copy(ctx, outs[j], in, r, 0);
        if (rc) return rc;
        off += sections[j];
    }
    return MTL_OK;
}

// SPLIT.backward (dynamics.mojo:166-199): the upper gradients of all outputs, side by side.
int32_t mtl_split_bwd(mtl_ctx* ctx, float* grad, const float* const* ugs, int32_t n_out, int32_t rank,
                      const int64_t* in_shape, const int64_t* sections, int32_t dim, int32_t accumulate) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, grad && ugs && sections && n_out >= 1 && shape_ok(rank, in_shape) && dim >= 0 && dim < rank,
                "bad arguments to mtl_split_bwd");
    int64_t total = 0, ist[MTL_MAX_RANK];
    for (int j = 0; j < n_out; ++j) { MTL_REQUIRE(ctx, sections[j] >= 1 && ugs[j], "bad section %d", j); total += sections[j]; }
    MTL_REQUIRE(ctx, total == in_shape[dim], "SPLIT sections sum to %lld, the axis has %lld", (long long)total, (long long)in_shape[dim]);
    contiguous_strides(rank, in_shape, ist);
    int64_t off = 0;
    for (int j = 0; j < n_out; ++j) {
        Region r;
        r.rank = rank; r.soff = 0; r.doff = off * ist[dim];
        for (int a = 0; a < rank; ++a) { r.shape[a] = a == dim ? sections[j] : in_shape[a]; r.ds[a] = ist[a]; }
        contiguous_strides(rank, r.shape, r.ss);
        int32_t rc = run_copy(ctx, grad, ugs[j], r, accumulate ? 1 : 0);
        if (rc) return rc;
        off += sections[j];
    }
    return MTL_OK;
}

}  // extern "C"
