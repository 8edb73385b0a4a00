// Data-parallel gradient exchange: one process per GPU, sum-allreduce of the flat gradient arena
// over NVLink through NCCL on a separate communication stream, event-ordered against the compute
// stream so that the exchange of a finished gradient bucket overlaps the backward pass of earlier
// layers.  NCCL is bound at run time (dlopen) so that single-GPU use needs no NCCL at all.
#include <stdlib.h>
#include <stdio.h>
#include <dlfcn.h>

#include <chrono>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <thread>

#include "common.cuh"

namespace {

// Minimal NCCL ABI (stable across 2.x): only the calls used here.
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclFloat32 = 7 };
enum { ncclSum = 0 };

struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(ncclUniqueId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*CommAbort)(ncclComm_t) = nullptr;
    int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
};

NcclApi g_nccl;

bool load_nccl(char* why, size_t why_len) {
    if (g_nccl.lib) return true;
    const char* names[] = {getenv("MANTLE_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* lib = nullptr;
    for (const char* n : names) {
        if (!n || !n[0]) continue;
        lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (lib) break;
    }
    if (!lib) {
        snprintf(why, why_len, "cannot load libnccl.so.2: %s", dlerror());
        return false;
    }
#define MTL_SYM(field, name)                                         \
    *(void**)(&g_nccl.field) = dlsym(lib, name);                     \
    if (!g_nccl.field) {                                             \
        snprintf(why, why_len, "libnccl lacks symbol %s", name);     \
        return false;                                                \
    }
    MTL_SYM(GetUniqueId, "ncclGetUniqueId")
    MTL_SYM(CommInitRank, "ncclCommInitRank")
    MTL_SYM(CommDestroy, "ncclCommDestroy")
    MTL_SYM(CommAbort, "ncclCommAbort")
    MTL_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
    MTL_SYM(AllReduce, "ncclAllReduce")
    MTL_SYM(Broadcast, "ncclBroadcast")
    MTL_SYM(GetErrorString, "ncclGetErrorString")
#undef MTL_SYM
    g_nccl.lib = lib;
    return true;
}

// Joining a group blocks inside the collective library until every rank has arrived; a rank that
// never arrives would block the others for ever.  The join therefore runs on a helper thread and the
// caller waits for it with a deadline.  When the deadline passes the caller gets MTL_ERR_COMM back;
// the helper stays blocked in the library (it cannot be interrupted before a communicator exists) and
// is left behind -- it holds no GPU work and ends with the process.  The shared record outlives
// whichever side finishes last.
struct JoinRecord {
    std::mutex mu;
    std::condition_variable cv;
    bool finished = false, abandoned = false;
    int result = 0;
    ncclComm_t comm = nullptr;
};

int join_timeout_ms() {
    const char* e = getenv("MANTLE_DP_INIT_TIMEOUT_S");
    double s = (e && *e) ? atof(e) : 120.0;
    if (s <= 0) s = 120.0;
    return (int)(s * 1000.0);
}

// Returns MTL_OK with *comm set, or MTL_ERR_COMM with the reason in `why`.  `device` >= 0 is made
// current on the helper thread (the library binds the communicator to the current device).
int32_t join_with_deadline(const ncclUniqueId& uid, int rank, int world, int device, int timeout_ms, ncclComm_t* comm,
                           char* why, size_t why_len) {
    auto rec = std::make_shared<JoinRecord>();
    std::thread([rec, uid, rank, world, device] {
        if (device >= 0) cudaSetDevice(device);
        ncclComm_t c = nullptr;
        int r = g_nccl.CommInitRank(&c, world, uid, rank);
        std::unique_lock<std::mutex> lk(rec->mu);
        if (rec->abandoned) {            // the caller gave up: nobody will use this communicator
            lk.unlock();
            if (r == ncclSuccess && c) g_nccl.CommAbort(c);
            return;
        }
        rec->result = r;
        rec->comm = c;
        rec->finished = true;
        rec->cv.notify_all();
    }).detach();
    std::unique_lock<std::mutex> lk(rec->mu);
    if (!rec->cv.wait_for(lk, std::chrono::milliseconds(timeout_ms), [&] { return rec->finished; })) {
        rec->abandoned = true;
        snprintf(why, why_len, "rank %d of %d: the group was not complete after %.1f s (a rank is late or missing); "
                 "set MANTLE_DP_INIT_TIMEOUT_S to wait longer", rank, world, timeout_ms / 1000.0);
        return MTL_ERR_COMM;
    }
    if (rec->result != ncclSuccess) {
        snprintf(why, why_len, "ncclCommInitRank failed: %s", g_nccl.GetErrorString(rec->result));
        return MTL_ERR_COMM;
    }
    *comm = rec->comm;
    return MTL_OK;
}

struct DpState {
    ncclComm_t comm = nullptr;
    bool failed = false;          // an asynchronous error was seen: the communicator is aborted, not destroyed
    int rank = 0, world = 1;
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t ready = nullptr;  // compute -> comm
    cudaEvent_t done = nullptr;   // comm -> compute
    bool pending = false;
    int reserved_sms = 0;         // SMs the compute kernels leave to the collective (taken off ctx->sm_count)
};

#define MTL_NCCL(ctx, call)                                                                      \
    do {                                                                                         \
        int r__ = (call);                                                                        \
        if (r__ != ncclSuccess)                                                                  \
            return mtl_set_error(ctx, MTL_ERR_COMM, "%s failed: %s", #call, g_nccl.GetErrorString(r__)); \
    } while (0)

}  // namespace

extern "C" {

int32_t mtl_dp_get_unique_id(uint8_t* out_id) {
    if (!out_id) return MTL_ERR_INVALID;
    char why[256];
    if (!load_nccl(why, sizeof(why))) {
        fprintf(stderr, "[mantle_cuda] %s\n", why);
        return MTL_ERR_COMM;
    }
    ncclUniqueId id;
    if (g_nccl.GetUniqueId(&id) != ncclSuccess) return MTL_ERR_COMM;
    static_assert(sizeof(id) == MTL_DP_ID_BYTES, "unique id size");
    memcpy(out_id, &id, MTL_DP_ID_BYTES);
    return MTL_OK;
}

int32_t mtl_dp_init(mtl_ctx* ctx, const uint8_t* id, int32_t rank, int32_t world) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, id && world >= 1 && rank >= 0 && rank < world, "bad arguments to mtl_dp_init");
    MTL_REQUIRE(ctx, !ctx->dp, "data-parallel group already initialised on this context");
    char why[256];
    if (!load_nccl(why, sizeof(why))) return mtl_set_error(ctx, MTL_ERR_COMM, "%s", why);
    MTL_CUDA(ctx, cudaSetDevice(ctx->device));
    DpState* st = new DpState();
    st->rank = rank;
    st->world = world;
    ncclUniqueId uid;
    memcpy(&uid, id, MTL_DP_ID_BYTES);
    // The tensor-core kernels are persistent: one CTA per SM that needs the SM's whole shared memory, tiles
    // dealt out in advance.  A collective kernel that holds a few SMs when such a kernel starts makes the
    // CTAs meant for those SMs start late, and the whole kernel ends late by as much (measured: +0.08 to
    // +0.10 ms per step at 2, 4 and 8 GPUs, far more than the exchange itself).  So the collective is
    // limited to a few CTAs and the compute kernels leave that many SMs free (below).
    // Measured at 2 GPUs, global batch 2048 / 512: 0.774 / 0.302 ms per step with nothing reserved, 0.739 /
    // 0.294 ms with 8 SMs reserved and at most 8 (or 4) collective CTAs, 0.755 ms with 16 reserved.
    int reserve = 8;
    if (const char* e = getenv("MANTLE_DP_RESERVE_SMS")) reserve = atoi(e);
    if (reserve < 0) reserve = 0;
    if (reserve > 0 && world > 1) {
        char buf[16];
        int ctas = reserve;
        if (const char* e = getenv("MANTLE_DP_NCCL_CTAS")) ctas = atoi(e) > 0 ? atoi(e) : reserve;
        snprintf(buf, sizeof(buf), "%d", ctas);
        setenv("NCCL_MAX_CTAS", buf, 0);   // a value set by the user wins
    }
    if (join_with_deadline(uid, rank, world, ctx->device, join_timeout_ms(), &st->comm, why, sizeof(why)) != MTL_OK) {
        delete st;
        return mtl_set_error(ctx, MTL_ERR_COMM, "%s", why);
    }
    int prio_lo = 0, prio_hi = 0;
    cudaDeviceGetStreamPriorityRange(&prio_lo, &prio_hi);
    if (cudaStreamCreateWithPriority(&st->comm_stream, cudaStreamNonBlocking, prio_hi) != cudaSuccess ||
        cudaEventCreateWithFlags(&st->ready, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&st->done, cudaEventDisableTiming) != cudaSuccess) {
        g_nccl.CommDestroy(st->comm);
        delete st;
        return mtl_set_error(ctx, MTL_ERR_CUDA, "could not create the communication stream");
    }
    ctx->dp = st;
    if (world > 1 && reserve > 0 && ctx->sm_count > 2 * reserve) {
        st->reserved_sms = reserve;
        ctx->sm_count -= reserve;          // persistent grids are sized from this
    }
    return MTL_OK;
}

int32_t mtl_dp_allreduce_async(mtl_ctx* ctx, float* buf, int64_t n) {
    MTL_CHECK_CTX(ctx);
    DpState* st = (DpState*)ctx->dp;
    MTL_REQUIRE(ctx, st, "mtl_dp_init has not been called");
    MTL_REQUIRE(ctx, buf && n >= 0, "bad arguments to mtl_dp_allreduce_async");
    if (st->failed) return mtl_set_error(ctx, MTL_ERR_COMM, "the communicator failed earlier and was aborted");
    if (n == 0 || st->world == 1) return MTL_OK;
    MTL_CUDA(ctx, cudaEventRecord(st->ready, ctx->stream));
    MTL_CUDA(ctx, cudaStreamWaitEvent(st->comm_stream, st->ready, 0));
    MTL_NCCL(ctx, g_nccl.AllReduce(buf, buf, (size_t)n, ncclFloat32, ncclSum, st->comm, st->comm_stream));
    st->pending = true;
    return MTL_OK;
}

int32_t mtl_dp_wait(mtl_ctx* ctx) {
    MTL_CHECK_CTX(ctx);
    DpState* st = (DpState*)ctx->dp;
    MTL_REQUIRE(ctx, st, "mtl_dp_init has not been called");
    if (!st->pending) return MTL_OK;
    MTL_CUDA(ctx, cudaEventRecord(st->done, st->comm_stream));
    MTL_CUDA(ctx, cudaStreamWaitEvent(ctx->stream, st->done, 0));
    st->pending = false;
    return MTL_OK;
}

int32_t mtl_dp_status(mtl_ctx* ctx) {
    MTL_CHECK_CTX(ctx);
    DpState* st = (DpState*)ctx->dp;
    MTL_REQUIRE(ctx, st, "mtl_dp_init has not been called");
    if (st->failed) return mtl_set_error(ctx, MTL_ERR_COMM, "the communicator failed earlier and was aborted");
    int async = ncclSuccess;
    int r = g_nccl.CommGetAsyncError(st->comm, &async);
    if (r == ncclSuccess && async == ncclSuccess) return MTL_OK;
    const int bad = r != ncclSuccess ? r : async;
    st->failed = true;
    g_nccl.CommAbort(st->comm);   // frees the library's resources without waiting for the peers
    st->comm = nullptr;
    return mtl_set_error(ctx, MTL_ERR_COMM, "asynchronous collective error: %s; the communicator was aborted",
                         g_nccl.GetErrorString(bad));
}

int32_t mtl_dp_probe(const uint8_t* id, int32_t rank, int32_t world, int32_t timeout_ms) {
    if (!id || world < 1 || rank < 0 || rank >= world || timeout_ms <= 0) return MTL_ERR_INVALID;
    char why[256];
    if (!load_nccl(why, sizeof(why))) {
        fprintf(stderr, "[mantle_cuda] %s\n", why);
        return MTL_ERR_COMM;
    }
    ncclUniqueId uid;
    memcpy(&uid, id, MTL_DP_ID_BYTES);
    ncclComm_t comm = nullptr;
    if (join_with_deadline(uid, rank, world, -1, timeout_ms, &comm, why, sizeof(why)) != MTL_OK) {
        fprintf(stderr, "[mantle_cuda] %s\n", why);
        return MTL_ERR_COMM;
    }
    g_nccl.CommDestroy(comm);
    return MTL_OK;
}

int32_t mtl_dp_broadcast(mtl_ctx* ctx, float* buf, int64_t n, int32_t root) {
    MTL_CHECK_CTX(ctx);
    DpState* st = (DpState*)ctx->dp;
    MTL_REQUIRE(ctx, st, "mtl_dp_init has not been called");
    MTL_REQUIRE(ctx, buf && n >= 0 && root >= 0 && root < st->world, "bad arguments to mtl_dp_broadcast");
    if (st->failed) return mtl_set_error(ctx, MTL_ERR_COMM, "the communicator failed earlier and was aborted");
    if (n == 0 || st->world == 1) return MTL_OK;
    MTL_NCCL(ctx, g_nccl.Broadcast(buf, buf, (size_t)n, ncclFloat32, root, st->comm, ctx->stream));
    return MTL_OK;
}

int32_t mtl_set_grads_ready_hook(mtl_ctx* ctx, void (*hook)(void* user), void* user) {
    MTL_CHECK_CTX(ctx);
    ctx->grads_ready_hook = hook;
    ctx->grads_ready_user = hook ? user : nullptr;
    return MTL_OK;
}

int32_t mtl_dp_world_size(mtl_ctx* ctx) {
    if (!ctx || !ctx->dp) return 1;
    return ((DpState*)ctx->dp)->world;
}

int32_t mtl_dp_destroy(mtl_ctx* ctx) {
    MTL_CHECK_CTX(ctx);
    DpState* st = (DpState*)ctx->dp;
    if (!st) return MTL_OK;
    cudaStreamSynchronize(st->comm_stream);
    cudaStreamSynchronize(ctx->stream);
    if (st->comm) g_nccl.CommDestroy(st->comm);
    cudaEventDestroy(st->ready);
    cudaEventDestroy(st->done);
    cudaStreamDestroy(st->comm_stream);
    ctx->sm_count += st->reserved_sms;
    delete st;
    ctx->dp = nullptr;
    return MTL_OK;
}

}  // extern "C"
