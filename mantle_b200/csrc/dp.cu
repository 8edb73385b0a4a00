// Data-parallel gradient exchange: one process per GPU, sum-allreduce of the flat gradient arena
// over NVLink through NCCL on a separate communication stream, event-ordered against the compute
// stream so that the exchange of a finished gradient bucket overlaps the backward pass of earlier
// layers.  NCCL is bound at run time (dlopen) so that single-GPU use needs no NCCL at all.
//
// The LAST bucket of a step cannot overlap anything: the gradients of the first layer are final only
// when the backward pass is over, and a library collective then costs its launch, its protocol and
// two stream hand-overs (measured: 35 - 43 us of a step exposed at 2 GPUs) for a few kilobytes.  For
// that bucket (mtl_dp_allreduce_tail) the ranks of one machine exchange directly over NVLink: every
// rank maps every other rank's exchange buffer (CUDA IPC) at start-up, and one kernel on the compute
// stream pushes its values into the peers' buffers as 8-byte {value, step number} words and then
// collects the peers' values from its own buffer, summing in rank order (every rank gets the same bits).
// The same kernel can carry the other buckets (up to 2 MB, channel 1 of the buffers, on the communication
// stream; MANTLE_DP_BUCKET_EXCHANGE=1).  It is light enough to run beside a persistent tensor-core CTA,
// which the library collective's CTAs are not -- but measured it loses to the library at that size: 2 GPUs
// 0.692 against 0.683 ms per step, 4 GPUs 0.431 against 0.407 ms (twice the bytes on the wire, and its
// polling shares SMs with the compute kernels).  So it is an opt-in and only the last bucket goes direct.
// An 8-byte store is indivisible, so a word whose step number matches carries its value: no flags, no
// fences.  Two buffer halves used in turn keep a fast rank's next step off the words a slow rank still
// reads (a rank cannot run two steps ahead: its next exchange needs the slow rank's push).  Every wait
// on a peer is bounded; when it runs out the kernel writes MTL_ERR_TIMEOUT to the status word, leaves
// the gradient as it was and returns.
#include <stdlib.h>
#include <stdio.h>
#include <dlfcn.h>

#include <chrono>
#include <condition_variable>
#include <memory>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"

namespace {

// Minimal NCCL ABI (stable across 2.x): only the calls used here.
typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0 };
enum { ncclInt8 = 0, ncclInt32 = 2, ncclFloat32 = 7 };
enum { ncclSum = 0, ncclMin = 3 };

struct NcclApi {
    void* lib = nullptr;
    int (*GetUniqueId)(ncclUniqueId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*CommAbort)(ncclComm_t) = nullptr;
    int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;   // optional
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
    *(void**)(&g_nccl.AllGather) = dlsym(lib, "ncclAllGather");   // without it the tail exchange stays off
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
    // direct exchange of the last bucket (see the top of this file)
    bool tail_on = false;
    uint2* xbuf = nullptr;        // this rank's buffer: per channel [2 halves][world][capacity] {value, step}
    uint2* peer_xbuf[8] = {};     // every rank's buffer as mapped here ([rank] = xbuf)
    uint32_t* ctl = nullptr;      // device, behind the words: per channel {exchanges done, ticket}
    bool bucket_direct = false;   // MANTLE_DP_BUCKET_EXCHANGE=1: the other buckets (up to 2 MB) go direct as well, on the communication stream
};

constexpr int kTailCap = 16384;           // channel 0 (compute stream): floats per exchange (64 KB of gradient)
constexpr int kBucketCap = 1 << 19;       // channel 1 (communication stream): 2 MB of gradient
constexpr int kTailMaxWorld = 8;
inline size_t chan_words(int world, int chan) { return (size_t)2 * world * (chan ? kBucketCap : kTailCap); }
inline size_t chan_offset(int world, int chan) { return chan ? chan_words(world, 0) : 0; }
constexpr uint64_t kTailBudgetNs = 20ull * 1000 * 1000 * 1000;

struct TailX {
    float* grad;
    int n, rank, world, cap;       // cap: floats per (half, rank) slot of this channel
    uint2* slots[kTailMaxWorld];   // slots[r]: rank r's buffer (this channel's part)
    uint32_t* seq;                 // exchanges done so far (this rank's counter)
    int32_t* ticket;               // zero between launches
    int32_t* status;
    uint64_t budget_ns;
};

__device__ __forceinline__ uint64_t tail_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_word(uint2* p, uint32_t value, uint32_t step) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(value), "r"(step) : "memory");
}
__device__ __forceinline__ uint2 ld_word(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}

// One rank's part of the exchange, run by `nblocks` blocks of 256 threads (block index `b` among them).
// A thread first pushes all its elements to every peer, then collects them from every peer: no thread waits
// for another thread of its own rank.  The polling loop naps between looks, so that a block that shares
// its SM with a tensor-core CTA takes few of its issue slots.
__device__ void tail_exchange_rank(const TailX& p, int b, int nblocks, bool silent) {
    __shared__ int s_last;
    const uint32_t step = *reinterpret_cast<volatile uint32_t*>(p.seq) + 1u;
    const int half = (int)(step & 1u);
    bool timed_out = false;
    const int first = b * 256 + (int)threadIdx.x, stride = nblocks * 256;
    if (!silent) {
        for (int i = first; i < p.n; i += stride) {
            const uint32_t g = __float_as_uint(p.grad[i]);
            for (int r = 0; r < p.world; ++r)
                if (r != p.rank) st_word(p.slots[r] + ((size_t)(half * p.world + p.rank) * p.cap + i), g, step);
        }
        const uint64_t t0 = tail_timer_ns();
        for (int i = first; i < p.n && !timed_out; i += stride) {
            const float g = p.grad[i];
            float sum = 0.0f;
            for (int r = 0; r < p.world && !timed_out; ++r) {
                float v = g;
                if (r != p.rank) {
                    const uint2* src = p.slots[p.rank] + ((size_t)(half * p.world + r) * p.cap + i);
                    uint2 w = ld_word(src);
                    for (uint32_t spins = 0; w.y != step; ++spins) {
                        if ((spins & 15u) == 15u && tail_timer_ns() - t0 > p.budget_ns) { timed_out = true; break; }
                        __nanosleep(64);
                        w = ld_word(src);
                    }
                    v = __uint_as_float(w.x);
                }
                sum += v;
            }
            if (!timed_out) p.grad[i] = sum;
        }
    }
    if (timed_out) atomicExch(p.status, MTL_ERR_TIMEOUT);
    // the block that finishes last counts the exchange (every block has read the counter by then)
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(p.ticket, 1) == nblocks - 1;
    __syncthreads();
    if (s_last && threadIdx.x == 0) {
        *reinterpret_cast<volatile uint32_t*>(p.seq) = step;
        *p.ticket = 0;
    }
}

__global__ void __launch_bounds__(256) k_tail_exchange(TailX p) {
    mtl_pdl_sync();
    tail_exchange_rank(p, (int)blockIdx.x, (int)gridDim.x, false);
}

// All ranks of a group in ONE launch on one GPU (self-test): blockIdx.y is the rank.  The blocks wait on
// one another, so the launch is cooperative (all blocks resident) and small.
struct TailXAll {
    TailX r[kTailMaxWorld];
    int silent_rank;   // a rank that never pushes (-1: none)
};
__global__ void __launch_bounds__(256) k_tail_exchange_all(TailXAll a) {
    tail_exchange_rank(a.r[blockIdx.y], (int)blockIdx.x, (int)gridDim.x, (int)blockIdx.y == a.silent_rank);
}

#define MTL_NCCL(ctx, call)                                                                      \
    do {                                                                                         \
        int r__ = (call);                                                                        \
        if (r__ != ncclSuccess)                                                                  \
            return mtl_set_error(ctx, MTL_ERR_COMM, "%s failed: %s", #call, g_nccl.GetErrorString(r__)); \
    } while (0)

void tail_release(DpState* st) {
    for (int r = 0; r < kTailMaxWorld; ++r) {
        if (st->peer_xbuf[r] && r != st->rank) cudaIpcCloseMemHandle(st->peer_xbuf[r]);
        st->peer_xbuf[r] = nullptr;
    }
    if (st->xbuf) cudaFree(st->xbuf);
    st->xbuf = nullptr;
    st->ctl = nullptr;
    st->tail_on = false;
}

}  // namespace

// Launches the direct exchange of `n` floats on `stream` through channel `chan` of the buffers.
static int32_t launch_direct(mtl_ctx* ctx, DpState* st, int chan, float* buf, int64_t n, cudaStream_t stream) {
    TailX p;
    p.grad = buf; p.n = (int)n; p.rank = st->rank; p.world = st->world;
    p.cap = chan ? kBucketCap : kTailCap;
    for (int r = 0; r < kTailMaxWorld; ++r) p.slots[r] = st->peer_xbuf[r] ? st->peer_xbuf[r] + chan_offset(st->world, chan) : nullptr;
    p.seq = st->ctl + 2 * chan;
    p.ticket = reinterpret_cast<int32_t*>(st->ctl + 2 * chan + 1);
    p.status = ctx->dev_status;
    p.budget_ns = kTailBudgetNs;
    const int64_t want = (n + 255) / 256;
    const int blocks = (int)(want < 64 ? want : 64);
    if (stream == ctx->stream) mtl_launch_pdl(ctx, k_tail_exchange, dim3(blocks), dim3(256), (size_t)0, p);
    else k_tail_exchange<<<blocks, 256, 0, stream>>>(p);
    MTL_LAUNCHED(ctx);
    return MTL_OK;
}

// Maps every rank's exchange buffer into this process.  Every rank runs the same collectives here, whether
// or not it wants (or manages) the direct exchange, and the group uses it only if EVERY rank mapped every
// buffer: a rank on its own would wait for pushes that never come.
static int32_t tail_setup(mtl_ctx* ctx, DpState* st, bool want) {
    const int W = st->world;
    const size_t words = chan_words(W, 0) + chan_words(W, 1);
    int ok = want ? 1 : 0;
    cudaIpcMemHandle_t mine;
    memset(&mine, 0, sizeof(mine));
    if (ok && (cudaMalloc(&st->xbuf, words * sizeof(uint2) + 256) != cudaSuccess ||
               cudaMemset(st->xbuf, 0, words * sizeof(uint2) + 256) != cudaSuccess ||
               cudaDeviceSynchronize() != cudaSuccess || cudaIpcGetMemHandle(&mine, st->xbuf) != cudaSuccess)) {
        cudaGetLastError();
        ok = 0;
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    uint8_t* dev = nullptr;   // [W handles][one int32 flag]
    MTL_CUDA(ctx, cudaMalloc(&dev, (size_t)(W + 1) * 64));
    std::unique_ptr<uint8_t, void (*)(uint8_t*)> dev_owner(dev, [](uint8_t* q) { cudaFree(q); });
    MTL_CUDA(ctx, cudaMemcpyAsync(dev + (size_t)st->rank * 64, &mine, 64, cudaMemcpyHostToDevice, ctx->stream));
    MTL_NCCL(ctx, g_nccl.AllGather(dev + (size_t)st->rank * 64, dev, 64, ncclInt8, st->comm, ctx->stream));
    std::vector<cudaIpcMemHandle_t> all((size_t)W);
    MTL_CUDA(ctx, cudaMemcpyAsync(all.data(), dev, (size_t)W * 64, cudaMemcpyDeviceToHost, ctx->stream));
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int r = 0; r < W && ok; ++r) {
        if (r == st->rank) { st->peer_xbuf[r] = st->xbuf; continue; }
        void* q = nullptr;
        if (cudaIpcOpenMemHandle(&q, all[(size_t)r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            ok = 0;
        } else {
            st->peer_xbuf[r] = (uint2*)q;
        }
    }
    int32_t flag = ok;
    int32_t* dflag = reinterpret_cast<int32_t*>(dev + (size_t)W * 64);
    MTL_CUDA(ctx, cudaMemcpyAsync(dflag, &flag, 4, cudaMemcpyHostToDevice, ctx->stream));
    MTL_NCCL(ctx, g_nccl.AllReduce(dflag, dflag, 1, ncclInt32, ncclMin, st->comm, ctx->stream));
    MTL_CUDA(ctx, cudaMemcpyAsync(&flag, dflag, 4, cudaMemcpyDeviceToHost, ctx->stream));
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (flag == 1) {
        st->tail_on = true;
        st->ctl = reinterpret_cast<uint32_t*>(st->xbuf + words);
    } else {
        tail_release(st);
    }
    return MTL_OK;
}

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
    // dealt out in advance, so a collective kernel can only run beside them on SMs they leave free.
    // MANTLE_DP_RESERVE_SMS = n makes every persistent grid n CTAs smaller and limits the collective to n
    // CTAs.  Measured with the kernels as they are now, global batch 2048 (ms per step, 0 / 8 reserved):
    // 2 GPUs 0.721 / 0.756, 4 GPUs 0.431 / 0.454, 4 GPUs at 256 images each 0.284 / 0.304 (and 0.325 with 4).
    // Leaving nothing free wins: the exchange of a bucket then runs in the gaps between the persistent
    // kernels and beside the lighter ones, and the compute kernels keep all SMs.
    int reserve = 0;
    if (const char* e = getenv("MANTLE_DP_RESERVE_SMS")) reserve = atoi(e);
    if (reserve < 0) reserve = 0;
    // Reserving only where it is free was measured too: a persistent grid launched WHILE an exchange is in
    // flight left 8 SMs to it when its tiles needed no extra wave for that (at 256 images per GPU conv2's input
    // gradient has 256 tiles: two waves on 148 SMs and on 140).  It lost as well -- 4 GPUs 0.428 against 0.407 ms
    // per step, 4 ranks at 256 images each 0.289 against 0.273: an all-reduce squeezed into 8 CTAs beside a
    // tensor-core kernel takes longer than one that waits for the kernel's end and then has the machine.
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
    int want_tail = 1;
    if (const char* e = getenv("MANTLE_DP_TAIL_EXCHANGE")) want_tail = atoi(e);
    if (const char* e = getenv("MANTLE_DP_BUCKET_EXCHANGE")) st->bucket_direct = atoi(e) != 0;
    if (world > 1 && world <= kTailMaxWorld && g_nccl.AllGather) {
        int32_t rc = tail_setup(ctx, st, want_tail != 0);
        if (rc) return rc;
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
    if (st->tail_on && st->bucket_direct && n <= kBucketCap)
    {   // fits beside the tensor-core kernels; see the top of this file
        int32_t rc = launch_direct(ctx, st, 1, buf, n, st->comm_stream);
        if (rc) return rc;
    } else
        MTL_NCCL(ctx, g_nccl.AllReduce(buf, buf, (size_t)n, ncclFloat32, ncclSum, st->comm, st->comm_stream));
    st->pending = true;
    return MTL_OK;
}

int32_t mtl_dp_allreduce_tail(mtl_ctx* ctx, float* buf, int64_t n) {
    MTL_CHECK_CTX(ctx);
    DpState* st = (DpState*)ctx->dp;
    MTL_REQUIRE(ctx, st, "mtl_dp_init has not been called");
    MTL_REQUIRE(ctx, buf && n >= 0, "bad arguments to mtl_dp_allreduce_tail");
    if (!st->tail_on || n > kTailCap) return mtl_dp_allreduce_async(ctx, buf, n);
    if (st->failed) return mtl_set_error(ctx, MTL_ERR_COMM, "the communicator failed earlier and was aborted");
    if (n == 0) return MTL_OK;
    return launch_direct(ctx, st, 0, buf, n, ctx->stream);
}

int32_t mtl_dp_tail_exchange_enabled(mtl_ctx* ctx) {
    if (!ctx || !ctx->dp) return 0;
    return ((DpState*)ctx->dp)->tail_on ? 1 : 0;
}

int32_t mtl_selftest_tail_exchange(mtl_ctx* ctx, float* grads, int32_t world, int32_t n, int32_t steps,
                                   int32_t silent_rank, int32_t budget_us) {
    MTL_CHECK_CTX(ctx);
    MTL_REQUIRE(ctx, grads && world >= 2 && world <= kTailMaxWorld && n >= 1 && n <= kTailCap && steps >= 1 &&
                         silent_rank < world && budget_us >= 1,
                "bad arguments to mtl_selftest_tail_exchange");
    int coop = 0;
    MTL_CUDA(ctx, cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
    MTL_REQUIRE(ctx, coop, "the device cannot launch cooperatively");
    const size_t words = chan_words(world, 0);
    const size_t per_rank = words * sizeof(uint2) + 256;
    uint8_t* mem = nullptr;
    MTL_CUDA(ctx, cudaMalloc(&mem, per_rank * world));
    std::unique_ptr<uint8_t, void (*)(uint8_t*)> owner(mem, [](uint8_t* q) { cudaFree(q); });
    MTL_CUDA(ctx, cudaMemsetAsync(mem, 0, per_rank * world, ctx->stream));
    TailXAll a;
    a.silent_rank = silent_rank;
    for (int r = 0; r < world; ++r) {
        TailX& p = a.r[r];
        p.grad = grads + (size_t)r * n; p.n = n; p.rank = r; p.world = world; p.cap = kTailCap;
        for (int q = 0; q < kTailMaxWorld; ++q) p.slots[q] = q < world ? reinterpret_cast<uint2*>(mem + per_rank * q) : nullptr;
        p.seq = reinterpret_cast<uint32_t*>(mem + per_rank * r + words * sizeof(uint2));
        p.ticket = reinterpret_cast<int32_t*>(p.seq) + 1;
        p.status = ctx->dev_status;
        p.budget_ns = (uint64_t)budget_us * 1000ull;
    }
    const int blocks = (n + 255) / 256 < 8 ? (n + 255) / 256 : 8;   // at most 64 blocks in all: resident together
    void* args[] = {&a};
    for (int s = 0; s < steps; ++s) {
        MTL_CUDA(ctx, cudaLaunchCooperativeKernel((void*)k_tail_exchange_all, dim3(blocks, world), dim3(256), args, 0, ctx->stream));
        MTL_LAUNCHED(ctx);
    }
    MTL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
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
    tail_release(st);
    cudaEventDestroy(st->ready);
    cudaEventDestroy(st->done);
    cudaStreamDestroy(st->comm_stream);
    ctx->sm_count += st->reserved_sms;
    delete st;
    ctx->dp = nullptr;
    return MTL_OK;
}

}  // extern "C"
