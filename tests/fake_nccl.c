/* A stand-in for libnccl used ONLY by tests/test_dp_failures_cpu.py: the handful of NCCL entry points
 * libmantle_cuda.so binds at run time, with the rendezvous done through files in a directory, so that
 * the host-side failure handling of the data-parallel group (a rank that joins late, a rank that
 * never joins) can be exercised on CPU ranks.  No collective arithmetic happens here.
 *
 * The unique id carries the directory; ncclCommInitRank creates <dir>/rank.<r> and then blocks until
 * all `nranks` files exist -- for ever if one never appears, which is what the real library does. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>
#include <sys/stat.h>

typedef struct { char internal[128]; } ncclUniqueId;
typedef struct fakeComm { int rank, nranks; char dir[120]; } * ncclComm_t;
#define API __attribute__((visibility("default")))

API int ncclGetUniqueId(ncclUniqueId* id) {
    const char* d = getenv("FAKE_NCCL_DIR");
    memset(id, 0, sizeof(*id));
    if (!d || strlen(d) >= 120) return 5; /* ncclInvalidUsage */
    strcpy(id->internal, d);
    return 0;
}

API int ncclCommInitRank(ncclComm_t* comm, int nranks, ncclUniqueId id, int rank) {
    char path[256];
    snprintf(path, sizeof(path), "%s/rank.%d", id.internal, rank);
    FILE* f = fopen(path, "w");
    if (!f) return 2; /* ncclSystemError */
    fclose(f);
    for (;;) {
        int present = 0;
        struct stat st;
        for (int r = 0; r < nranks; ++r) {
            snprintf(path, sizeof(path), "%s/rank.%d", id.internal, r);
            present += stat(path, &st) == 0;
        }
        if (present == nranks) break;
        usleep(5000);
    }
    ncclComm_t c = (ncclComm_t)calloc(1, sizeof(**comm));
    c->rank = rank;
    c->nranks = nranks;
    strcpy(c->dir, id.internal);
    *comm = c;
    return 0;
}

API int ncclCommDestroy(ncclComm_t c) { free(c); return 0; }
API int ncclCommAbort(ncclComm_t c) {
    char path[256];
    snprintf(path, sizeof(path), "%s/aborted.%d", c->dir, c->rank);
    FILE* f = fopen(path, "w");
    if (f) fclose(f);
    free(c);
    return 0;
}
/* <dir>/async_error holds the error code the "network" reports, if the file exists */
API int ncclCommGetAsyncError(ncclComm_t c, int* err) {
    char path[256];
    snprintf(path, sizeof(path), "%s/async_error", c->dir);
    FILE* f = fopen(path, "r");
    *err = 0;
    if (f) {
        if (fscanf(f, "%d", err) != 1) *err = 6;
        fclose(f);
    }
    return 0;
}
API int ncclAllReduce(const void* s, void* r, size_t n, int t, int op, ncclComm_t c, void* stream) { return 0; }
API int ncclBroadcast(const void* s, void* r, size_t n, int t, int root, ncclComm_t c, void* stream) { return 0; }
API const char* ncclGetErrorString(int e) { return e == 0 ? "no error" : e == 6 ? "remote process exited or there was a network error" : "fake error"; }
