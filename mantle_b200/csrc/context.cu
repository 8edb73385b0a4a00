// Context, memory, stream-capture and timing entry points of libmantle_cuda.so.
#include <stdarg.h>

#include "common.cuh"

// guard zones of the debug allocator (see mtl_debug_check)
static constexpr size_t kGuardBytes = 256;
static constexpr int kGuardByte = 0xA5;

int32_t mtl_set_error(mtl_ctx* ctx, int32_t code, const char* fmt, ...) {
    if (ctx) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
        va_end(ap);
        if (ctx->tune.log_errors) fprintf(stderr, "[mantle_cuda] error %d: %s\n", code, ctx->err);
    }
    return code;
}

// Replaces a scratch block by a larger one.  The stream is drained first; the old block is freed
// unless an instantiated graph of this context may still name it, in which case it is parked until
// the last such graph is destroyed (a replayed step keeps using the block it was captured with).
static int32_t grow_block(mtl_ctx* ctx, void** block, size_t* have, size_t bytes, const char* what) {
    if (ctx->capturing)
        return mtl_set_error(ctx, MTL_ERR_NOMEM,
                             "%s of %zu bytes needed during stream capture but only %zu reserved; run the step "
                             "once (or call mtl_ctx_reserve_workspace) before capturing it",
                             what, bytes, *have);
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    size_t want = (bytes + (size_t)(1 << 20) - 1) & ~((size_t)(1 << 20) - 1);
    void* fresh = nullptr;
    if (*block && ctx->live_graphs == 0) {
        MTL_CUDA(ctx, cudaFree(*block));
        *block = nullptr;
        *have = 0;
    }
    cudaError_t e = cudaMalloc(&fresh, want);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return mtl_set_error(ctx, MTL_ERR_NOMEM, "cudaMalloc of %zu %s bytes failed: %s", want, what,
                             cudaGetErrorString(e));
    }
    if (*block) ctx->retired.push_back(*block);  // still named by a live graph
    *block = fresh;
    *have = want;
    return MTL_OK;
}

void mtl_release_retired(mtl_ctx* ctx) {
    if (ctx->live_graphs > 0) return;
    for (void* p : ctx->retired) cudaFree(p);
    ctx->retired.clear();
}

static int env_int(const char* name, int unset) {
    const char* e = getenv(name);
    return (e && *e) ? atoi(e) : unset;
}

static void read_tuning(mtl_tuning* t) {  // the only place the library reads its environment switches
    const char* log = getenv("MANTLE_CUDA_LOG");
    t->log_errors = log && log[0] == '1';
    t->conv_channel_major = env_int("MANTLE_CONV_CHANNEL_MAJOR", 1) != 0;
    t->conv_paired = env_int("MANTLE_CONV_PAIRED", 1) != 0;
    t->conv_spread = env_int("MANTLE_CONV_SPREAD", 1) != 0;
    t->conv_paired_min_kblocks = env_int("MANTLE_CONV_PAIRED_MIN_KB", 32);
    t->conv_tail_split = env_int("MANTLE_CONV_TAIL_SPLIT", 0) != 0;
    t->conv_pool_epilogue = env_int("MANTLE_CONV_POOL_EPILOGUE", 1) != 0;
    t->conv_first_tc = env_int("MANTLE_CONV_FIRST_TC", 1) != 0;
    t->gemm_3d_boxes = getenv("MANTLE_GEMM_NO3D") == nullptr;
    t->wgrad_taps = env_int("MANTLE_WGRAD_TAPS", -1);
    t->gemm_bn = env_int("MANTLE_GEMM_BN", -1);
    t->gemm_mt = env_int("MANTLE_GEMM_MT", -1);
    t->gemm_stages = env_int("MANTLE_GEMM_STAGES", -1);
    t->gemm_split_k = env_int("MANTLE_GEMM_SPLITK", -1);
    t->pdl = env_int("MANTLE_PDL", 1) != 0;
    t->debug_guards = env_int("MANTLE_CUDA_DEBUG", 0) != 0;
}

const mtl_tuning& mtl_global_tuning() {
    static const mtl_tuning t = [] { mtl_tuning v; read_tuning(&v); return v; }();
    return t;
}

int32_t mtl_workspace(mtl_ctx* ctx, size_t bytes, void** out) {
    if (bytes > ctx->ws_bytes) {
        int32_t rc = grow_block(ctx, &ctx->ws, &ctx->ws_bytes, bytes, "workspace");
        if (rc) return rc;
    }
    *out = ctx->ws;
    return MTL_OK;
}

// Room for one partial accumulator tile (128 rows x 256 fp32 columns) per SM: what the implicit-GEMM
// kernels need when the tiles of a partial last wave are split along k over two CTAs each.  Allocated
// once, never moved, so that captured graphs may keep naming it.
int32_t mtl_split_scratch(mtl_ctx* ctx, void** out) {
    if (!ctx->split_scratch) {
        const size_t want = (size_t)ctx->sm_count_total * 128 * 256 * 4;
        cudaError_t e = cudaMalloc(&ctx->split_scratch, want);
        if (e != cudaSuccess) {
            cudaGetLastError();
            ctx->split_scratch = nullptr;
            return mtl_set_error(ctx, MTL_ERR_NOMEM, "cudaMalloc of %zu split-scratch bytes failed: %s", want, cudaGetErrorString(e));
        }
    }
    *out = ctx->split_scratch;
    return MTL_OK;
}

// A second scratch block for callers that run other library kernels (which use the first one)
// on the data they keep here; same growth rules.
int32_t mtl_workspace2(mtl_ctx* ctx, size_t bytes, void** out) {
    if (bytes > ctx->ws2_bytes) {
        int32_t rc = grow_block(ctx, &ctx->ws2, &ctx->ws2_bytes, bytes, "scratch");
        if (rc) return rc;
    }
    *out = ctx->ws2;
    return MTL_OK;
}

extern "C" {

const char* mtl_version(void) { return "mantle_cuda 0.1 (sm_100a)"; }

int32_t mtl_ctx_create(int32_t device, mtl_ctx** out) {
    if (!out) return MTL_ERR_INVALID;
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count <= 0 || device < 0 || device >= count) {
        cudaGetLastError();
        return MTL_ERR_CUDA;  // no CPU fallback: without a device there is no context
    }
    if (cudaSetDevice(device) != cudaSuccess) return MTL_ERR_CUDA;
    mtl_ctx* ctx = new mtl_ctx();
    ctx->device = device;
    ctx->tune = mtl_global_tuning();
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        delete ctx;
        return MTL_ERR_CUDA;
    }
    ctx->owns_stream = true;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) == cudaSuccess) ctx->sm_count = ctx->sm_count_total = prop.multiProcessorCount;
    const size_t status_bytes = 256 + 8192 * sizeof(int32_t);
    if (cudaMalloc((void**)&ctx->dev_status, status_bytes) != cudaSuccess ||
        cudaMemset(ctx->dev_status, 0, status_bytes) != cudaSuccess) {
        cudaStreamDestroy(ctx->stream);
        delete ctx;
        return MTL_ERR_CUDA;
    }
    ctx->tickets = ctx->dev_status + 64;
    const char* mode = getenv("MANTLE_CUDA_MATH");
    if (mode) {
        if (!strcmp(mode, "fp32")) ctx->math_mode = MTL_MATH_FP32;
        else if (!strcmp(mode, "tf32")) ctx->math_mode = MTL_MATH_TF32;
        else if (!strcmp(mode, "tf32x3")) ctx->math_mode = MTL_MATH_TF32X3;
    }
    *out = ctx;
    return MTL_OK;
}

int32_t mtl_ctx_destroy(mtl_ctx* ctx) {
    MTL_CHECK_CTX(ctx);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->dp) mtl_dp_destroy(ctx);
    for (int k = 0; k < MTL_PROF_KERNELS; ++k)
        for (auto& ev : ctx->prof_events[k]) {
            cudaEventDestroy(ev.first);
            cudaEventDestroy(ev.second);
        }
    for (int i = 0; i < MTL_NUM_TIMERS; ++i) {
        if (ctx->t0[i]) cudaEventDestroy(ctx->t0[i]);
        if (ctx->t1[i]) cudaEventDestroy(ctx->t1[i]);
    }
    for (int i = 0; i < 4; ++i) {
        if (ctx->stage_ready[i]) cudaEventDestroy(ctx->stage_ready[i]);
        if (ctx->stage_free[i]) cudaEventDestroy(ctx->stage_free[i]);
    }
    if (ctx->copy_stream) {
        cudaStreamSynchronize(ctx->copy_stream);
        cudaStreamDestroy(ctx->copy_stream);
    }
    if (ctx->ws) cudaFree(ctx->ws);
    if (ctx->ws2) cudaFree(ctx->ws2);
    if (ctx->split_scratch) cudaFree(ctx->split_scratch);
    for (void* p : ctx->retired) cudaFree(p);
    for (auto& g : ctx->guarded) cudaFree((uint8_t*)g.first - kGuardBytes);   // blocks the caller never freed
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return MTL_OK;
}

int32_t mtl_ctx_set_stream(mtl_ctx* ctx, void* cuda_stream) {
    MTL_CHECK_CTX(ctx);
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->owns_stream && ctx->stream) cudaStreamDestroy(ctx->stream);
    ctx->stream = (cudaStream_t)cuda_stream;
    ctx->owns_stream = false;
    return MTL_OK;
}

void* mtl_ctx_stream(mtl_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int32_t mtl_ctx_set_math_mode(mtl_ctx* ctx, int32_t mode) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, mode >= MTL_MATH_FP32 && mode <= MTL_MATH_TF32X3, "unknown math mode %d", mode);
    ctx->math_mode = mode;
    return MTL_OK;
}

int32_t mtl_ctx_math_mode(mtl_ctx* ctx) { return ctx ? ctx->math_mode : -1; }

int32_t mtl_ctx_reserve_workspace(mtl_ctx* ctx, size_t bytes) {
    MTL_CHECK_CTX(ctx);
    void* p;
    return mtl_workspace(ctx, bytes, &p);
}

int32_t mtl_ctx_workspace_info(mtl_ctx* ctx, size_t* bytes, void** block, int32_t* live_graphs, int32_t* retired_blocks) {
    MTL_CHECK_CTX(ctx);
    if (bytes) *bytes = ctx->ws_bytes;
    if (block) *block = ctx->ws;
    if (live_graphs) *live_graphs = ctx->live_graphs;
    if (retired_blocks) *retired_blocks = (int32_t)ctx->retired.size();
    return MTL_OK;
}

int32_t mtl_sync(mtl_ctx* ctx) {
    MTL_CHECK_CTX(ctx);
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->tune.debug_guards && !ctx->capturing) return mtl_debug_check(ctx);
    return MTL_OK;
}

const char* mtl_last_error(mtl_ctx* ctx) { return ctx ? ctx->err : "null context"; }

int64_t mtl_launch_count(mtl_ctx* ctx) { return ctx ? ctx->launches : -1; }
int64_t mtl_conv_split_tiles(mtl_ctx* ctx) { return ctx ? ctx->conv_split_tiles : -1; }

int32_t mtl_device_status(mtl_ctx* ctx, int32_t* out_status) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, out_status, "null out_status");
    MTL_CUDA(ctx, cudaMemcpyAsync(out_status, ctx->dev_status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (*out_status != 0) MTL_CUDA(ctx, cudaMemsetAsync(ctx->dev_status, 0, 4, ctx->stream));
    return MTL_OK;
}

// ------------------------------------------------------------------ memory ---------------

// Debug guards (MANTLE_CUDA_DEBUG=1): every mtl_malloc block is placed between two 256-byte guard
// zones filled with a byte pattern.  A kernel that writes a little past either end of a tensor then
// damages a guard instead of a neighbouring allocation, and mtl_debug_check (called by mtl_sync and
// mtl_free in this mode) names the block: which allocation, which side, at which byte.

static int32_t check_guards(mtl_ctx* ctx, void* only) {
    uint8_t host[2 * kGuardBytes];
    for (size_t i = 0; i < ctx->guarded.size(); ++i) {
        uint8_t* user = (uint8_t*)ctx->guarded[i].first;
        if (only && user != only) continue;
        const size_t bytes = ctx->guarded[i].second;
        const size_t back_off = (bytes + 15) & ~(size_t)15;   // the rear guard starts at the next 16-byte boundary
        MTL_CUDA(ctx, cudaMemcpy(host, user - kGuardBytes, kGuardBytes, cudaMemcpyDeviceToHost));
        MTL_CUDA(ctx, cudaMemcpy(host + kGuardBytes, user + back_off, kGuardBytes, cudaMemcpyDeviceToHost));
        for (size_t b = 0; b < 2 * kGuardBytes; ++b) {
            if (host[b] == (uint8_t)kGuardByte) continue;
            const bool front = b < kGuardBytes;
            return mtl_set_error(ctx, MTL_ERR_INVALID,
                                 "guard damaged: allocation #%zu (%zu bytes at %p) was written %s it, %zu bytes %s",
                                 i, bytes, (void*)user, front ? "before" : "after",
                                 front ? kGuardBytes - b : b - kGuardBytes + (back_off - bytes), front ? "before its start" : "past its end");
        }
    }
    return MTL_OK;
}

int32_t mtl_malloc(mtl_ctx* ctx, size_t bytes, void** out_dptr) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, out_dptr, "null out pointer");
    *out_dptr = nullptr;
    if (bytes == 0) bytes = 4;
    const bool guard = ctx->tune.debug_guards;
    const size_t back_off = (bytes + 15) & ~(size_t)15;
    void* raw = nullptr;
    cudaError_t e = cudaMalloc(&raw, guard ? back_off + 2 * kGuardBytes : bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return mtl_set_error(ctx, MTL_ERR_NOMEM, "cudaMalloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    }
    if (guard) {
        MTL_CUDA(ctx, cudaMemset(raw, kGuardByte, kGuardBytes));
        MTL_CUDA(ctx, cudaMemset((uint8_t*)raw + kGuardBytes + back_off, kGuardByte, kGuardBytes));
        raw = (uint8_t*)raw + kGuardBytes;
        ctx->guarded.push_back({raw, bytes});
    }
    *out_dptr = raw;
    return MTL_OK;
}

int32_t mtl_free(mtl_ctx* ctx, void* dptr) {
    MTL_CHECK_CTX(ctx);
    if (!dptr) return MTL_OK;
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (ctx->tune.debug_guards) {
        for (size_t i = 0; i < ctx->guarded.size(); ++i) {
            if (ctx->guarded[i].first != dptr) continue;
            int32_t rc = check_guards(ctx, dptr);
            ctx->guarded.erase(ctx->guarded.begin() + (long)i);
            cudaFree((uint8_t*)dptr - kGuardBytes);
            return rc;
        }
    }
    MTL_CUDA(ctx, cudaFree(dptr));
    return MTL_OK;
}

int32_t mtl_debug_check(mtl_ctx* ctx) {
    MTL_CHECK_CTX(ctx);
    if (!ctx->tune.debug_guards) return MTL_OK;
    MTL_REQUIRE(ctx, !ctx->capturing, "guards cannot be checked during stream capture");
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return check_guards(ctx, nullptr);
}

int32_t mtl_h2d(mtl_ctx* ctx, void* dst, const void* src_host, size_t bytes) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, (dst && src_host) || bytes == 0, "null pointer in mtl_h2d");
    if (bytes == 0) return MTL_OK;
    MTL_CUDA(ctx, cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    // pageable sources are staged by the runtime before the call returns; pinned ones are not,
    // so wait: the caller may reuse the buffer as soon as this returns.
    if (!ctx->capturing) MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MTL_OK;
}

int32_t mtl_d2h(mtl_ctx* ctx, void* dst_host, const void* src, size_t bytes) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, (dst_host && src) || bytes == 0, "null pointer in mtl_d2h");
    MTL_REQUIRE(ctx, !ctx->capturing, "mtl_d2h waits for the stream and cannot be captured");
    if (bytes) MTL_CUDA(ctx, cudaMemcpyAsync(dst_host, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return MTL_OK;
}

int32_t mtl_h2d_async(mtl_ctx* ctx, void* dst, const void* src_host, size_t bytes) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, (dst && src_host) || bytes == 0, "null pointer in mtl_h2d_async");
    if (bytes) MTL_CUDA(ctx, cudaMemcpyAsync(dst, src_host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return MTL_OK;
}

int32_t mtl_d2h_async(mtl_ctx* ctx, void* dst_host, const void* src, size_t bytes) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, (dst_host && src) || bytes == 0, "null pointer in mtl_d2h_async");
    if (bytes) MTL_CUDA(ctx, cudaMemcpyAsync(dst_host, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return MTL_OK;
}

static int32_t stage_setup(mtl_ctx* ctx, int32_t slot) {
    MTL_REQUIRE(ctx, slot >= 0 && slot < 4, "staging slot %d out of range", slot);
    if (!ctx->copy_stream) MTL_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking));
    if (!ctx->stage_ready[slot]) {
        MTL_CUDA(ctx, cudaEventCreateWithFlags(&ctx->stage_ready[slot], cudaEventDisableTiming));
        MTL_CUDA(ctx, cudaEventCreateWithFlags(&ctx->stage_free[slot], cudaEventDisableTiming));
    }
    return MTL_OK;
}

int32_t mtl_stage_h2d(mtl_ctx* ctx, int32_t slot, void* dst_dev, const void* src_host, size_t bytes) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, !ctx->capturing, "staged copies cannot be part of a captured step");
    int32_t rc = stage_setup(ctx, slot);
    if (rc) return rc;
    MTL_REQUIRE(ctx, (dst_dev && src_host) || bytes == 0, "null pointer in mtl_stage_h2d");
    if (ctx->stage_released[slot]) {
        MTL_CUDA(ctx, cudaStreamWaitEvent(ctx->copy_stream, ctx->stage_free[slot], 0));
        ctx->stage_released[slot] = false;
    }
    if (bytes) MTL_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, bytes, cudaMemcpyHostToDevice, ctx->copy_stream));
    return MTL_OK;
}

int32_t mtl_stage_acquire(mtl_ctx* ctx, int32_t slot) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, !ctx->capturing, "staged copies cannot be part of a captured step");
    int32_t rc = stage_setup(ctx, slot);
    if (rc) return rc;
    MTL_CUDA(ctx, cudaEventRecord(ctx->stage_ready[slot], ctx->copy_stream));
    MTL_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, ctx->stage_ready[slot], 0));
    return MTL_OK;
}

int32_t mtl_stage_release(mtl_ctx* ctx, int32_t slot) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, !ctx->capturing, "staged copies cannot be part of a captured step");
    int32_t rc = stage_setup(ctx, slot);
    if (rc) return rc;
    MTL_CUDA(ctx, cudaEventRecord(ctx->stage_free[slot], ctx->stream));
    ctx->stage_released[slot] = true;
    return MTL_OK;
}

int32_t mtl_host_alloc(mtl_ctx* ctx, size_t bytes, void** out_hptr) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, out_hptr, "null out pointer");
    cudaError_t e = cudaHostAlloc(out_hptr, bytes ? bytes : 4, cudaHostAllocDefault);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return mtl_set_error(ctx, MTL_ERR_NOMEM, "cudaHostAlloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    }
    return MTL_OK;
}

int32_t mtl_host_free(mtl_ctx* ctx, void* hptr) {
    MTL_CHECK_CTX(ctx);
    if (hptr) MTL_CUDA(ctx, cudaFreeHost(hptr));
    return MTL_OK;
}

int32_t mtl_zero(mtl_ctx* ctx, void* dptr, size_t bytes) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, dptr || bytes == 0, "null pointer in mtl_zero");
    if (bytes) MTL_CUDA(ctx, cudaMemsetAsync(dptr, 0, bytes, ctx->stream));
    return MTL_OK;
}

// ------------------------------------------------------------------ capture --------------

int32_t mtl_graph_begin(mtl_ctx* ctx) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, !ctx->capturing, "capture already in progress");
    MTL_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
    ctx->capturing = true;
    ctx->launches_at_capture = ctx->launches;
    return MTL_OK;
}

int32_t mtl_graph_end(mtl_ctx* ctx, mtl_graph** out) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, ctx->capturing, "no capture in progress");
    MTL_REQUIRE(ctx, out, "null out pointer");
    ctx->capturing = false;
    cudaGraph_t g = nullptr;
    MTL_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &g));
    cudaGraphExec_t exec = nullptr;
    cudaError_t e = cudaGraphInstantiate(&exec, g, 0);
    if (e != cudaSuccess) {
        cudaGraphDestroy(g);
        cudaGetLastError();
        return mtl_set_error(ctx, MTL_ERR_CUDA, "cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
    }
    mtl_graph* mg = new mtl_graph();
    mg->graph = g;
    mg->exec = exec;
    mg->launches = ctx->launches - ctx->launches_at_capture;
    ctx->live_graphs += 1;
    // captured launches did not run: they are counted each time the graph is launched
    ctx->launches = ctx->launches_at_capture;
    *out = mg;
    return MTL_OK;
}

int32_t mtl_graph_launch(mtl_ctx* ctx, mtl_graph* g) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, g && g->exec, "null graph");
    MTL_CUDA(ctx, cudaGraphLaunch(g->exec, ctx->stream));
    ctx->launches += g->launches;
    return MTL_OK;
}

int32_t mtl_graph_destroy(mtl_ctx* ctx, mtl_graph* g) {
    MTL_CHECK_CTX(ctx);
    if (!g) return MTL_OK;
    cudaStreamSynchronize(ctx->stream);
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
    if (ctx->live_graphs > 0) ctx->live_graphs -= 1;
    mtl_release_retired(ctx);
    return MTL_OK;
}

// ------------------------------------------------------------------ kernel profile -------

static void prof_clear(mtl_ctx* ctx) {
    for (auto& r : ctx->ranges) {
        cudaEventDestroy(r.e0);
        cudaEventDestroy(r.e1);
    }
    ctx->ranges.clear();
    if (ctx->range_open) {
        cudaEventDestroy(ctx->open_range.e0);
        cudaEventDestroy(ctx->open_range.e1);
        ctx->range_open = false;
    }
    for (int k = 0; k < MTL_PROF_KERNELS; ++k) {
        for (auto& ev : ctx->prof_events[k]) {
            cudaEventDestroy(ev.first);
            cudaEventDestroy(ev.second);
        }
        ctx->prof_events[k].clear();
    }
}

int32_t mtl_prof_enable(mtl_ctx* ctx, int32_t on) {
    MTL_CHECK_CTX(ctx);
    ctx->prof_on = on != 0;
    return MTL_OK;
}

int32_t mtl_prof_reset(mtl_ctx* ctx) {
    MTL_CHECK_CTX(ctx);
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    prof_clear(ctx);
    return MTL_OK;
}

int32_t mtl_prof_get(mtl_ctx* ctx, int32_t which, float* total_ms, int32_t* launches) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, which >= 0 && which < MTL_PROF_KERNELS && total_ms && launches, "bad profile query");
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    float sum = 0.0f;
    for (auto& ev : ctx->prof_events[which]) {
        float ms = 0.0f;
        MTL_CUDA(ctx, cudaEventElapsedTime(&ms, ev.first, ev.second));
        sum += ms;
    }
    *total_ms = sum;
    *launches = (int32_t)ctx->prof_events[which].size();
    return MTL_OK;
}

int32_t mtl_prof_range_begin(mtl_ctx* ctx, int32_t tag) {
    MTL_CHECK_CTX(ctx);
    if (!ctx->prof_on || ctx->capturing) return MTL_OK;   // events cannot be read back from a captured step
    MTL_REQUIRE(ctx, !ctx->range_open, "mtl_prof_range_begin: range %d is still open", ctx->open_range.tag);
    mtl_ctx::prof_range r = {tag, nullptr, nullptr, ctx->launches};
    MTL_CUDA(ctx, cudaEventCreate(&r.e0));
    MTL_CUDA(ctx, cudaEventCreate(&r.e1));
    MTL_CUDA(ctx, cudaEventRecord(r.e0, ctx->stream));
    ctx->open_range = r;
    ctx->range_open = true;
    return MTL_OK;
}

int32_t mtl_prof_range_end(mtl_ctx* ctx) {
    MTL_CHECK_CTX(ctx);
    if (!ctx->range_open) return MTL_OK;
    MTL_CUDA(ctx, cudaEventRecord(ctx->open_range.e1, ctx->stream));
    ctx->open_range.launches = ctx->launches - ctx->open_range.launches;
    ctx->ranges.push_back(ctx->open_range);
    ctx->range_open = false;
    return MTL_OK;
}

int32_t mtl_prof_range_count(mtl_ctx* ctx, int32_t* out_n) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, out_n, "null out pointer");
    *out_n = (int32_t)ctx->ranges.size();
    return MTL_OK;
}

int32_t mtl_prof_range_get(mtl_ctx* ctx, int32_t i, int32_t* tag, float* ms, int32_t* launches) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, i >= 0 && (size_t)i < ctx->ranges.size() && tag && ms && launches, "bad range query");
    const auto& r = ctx->ranges[(size_t)i];
    MTL_CUDA(ctx, cudaEventSynchronize(r.e1));
    MTL_CUDA(ctx, cudaEventElapsedTime(ms, r.e0, r.e1));
    *tag = r.tag;
    *launches = (int32_t)r.launches;
    return MTL_OK;
}

int32_t mtl_prof_dump(mtl_ctx* ctx, const char* path) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, path, "null path");
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    FILE* f = fopen(path, "w");
    if (!f) return mtl_set_error(ctx, MTL_ERR_INVALID, "cannot open %s for writing", path);
    // one line per tag in order of first appearance: ranges, kernel launches, total and mean device time
    std::vector<int32_t> tags;
    std::vector<double> total;
    std::vector<int64_t> count, launches;
    for (auto& r : ctx->ranges) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, r.e0, r.e1) != cudaSuccess) { cudaGetLastError(); ms = 0.0f; }
        size_t k = 0;
        while (k < tags.size() && tags[k] != r.tag) ++k;
        if (k == tags.size()) { tags.push_back(r.tag); total.push_back(0); count.push_back(0); launches.push_back(0); }
        total[k] += ms; count[k] += 1; launches[k] += r.launches;
    }
    double sum = 0;
    for (double t : total) sum += t;
    fprintf(f, "tag,ranges,kernel_launches,total_ms,mean_ms,percent\n");
    for (size_t k = 0; k < tags.size(); ++k)
        fprintf(f, "%d,%lld,%lld,%.6f,%.6f,%.3f\n", tags[k], (long long)count[k], (long long)launches[k], total[k],
                total[k] / (double)count[k], sum > 0 ? 100.0 * total[k] / sum : 0.0);
    static const char* names[MTL_PROF_KERNELS] = {"dot_tc", "conv_igemm", "conv_wgrad", "conv_first"};
    for (int k = 0; k < MTL_PROF_KERNELS; ++k) {
        double t = 0;
        for (auto& ev : ctx->prof_events[k]) {
            float ms = 0.0f;
            if (cudaEventElapsedTime(&ms, ev.first, ev.second) == cudaSuccess) t += ms; else cudaGetLastError();
        }
        if (!ctx->prof_events[k].empty())
            fprintf(f, "kernel:%s,%zu,%zu,%.6f,%.6f,\n", names[k], ctx->prof_events[k].size(), ctx->prof_events[k].size(), t,
                    t / (double)ctx->prof_events[k].size());
    }
    fclose(f);
    return MTL_OK;
}

// ------------------------------------------------------------------ timing ---------------

int32_t mtl_timer_start(mtl_ctx* ctx, int32_t slot) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, slot >= 0 && slot < MTL_NUM_TIMERS, "timer slot %d out of range", slot);
    if (!ctx->t0[slot]) {
        MTL_CUDA(ctx, cudaEventCreate(&ctx->t0[slot]));
        MTL_CUDA(ctx, cudaEventCreate(&ctx->t1[slot]));
    }
    MTL_CUDA(ctx, cudaEventRecord(ctx->t0[slot], ctx->stream));
    return MTL_OK;
}

int32_t mtl_timer_stop(mtl_ctx* ctx, int32_t slot) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, slot >= 0 && slot < MTL_NUM_TIMERS && ctx->t1[slot], "timer slot %d not started", slot);
    MTL_CUDA(ctx, cudaEventRecord(ctx->t1[slot], ctx->stream));
    return MTL_OK;
}

int32_t mtl_timer_elapsed_ms(mtl_ctx* ctx, int32_t slot, float* out_ms) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, slot >= 0 && slot < MTL_NUM_TIMERS && ctx->t1[slot] && out_ms, "bad timer query");
    MTL_CUDA(ctx, cudaEventSynchronize(ctx->t1[slot]));
    MTL_CUDA(ctx, cudaEventElapsedTime(out_ms, ctx->t0[slot], ctx->t1[slot]));
    return MTL_OK;
}

}  // extern "C"
