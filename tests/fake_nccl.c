/*
 * A stand-in for libnccl, for the failure-path tests of the communicator (test infrastructure only).
 * The library under test binds NCCL by name at run time (environment variable SYNAPTIK_NCCL_LIBRARY),
 * so a file that exports the same entry points can play a peer that never answers without any GPU
 * misbehaving: ncclAllReduce enqueues a HOST function on the given stream that sleeps for
 * FAKE_NCCL_STALL_MS milliseconds or until ncclCommAbort is called (the stream is blocked, the GPU is
 * idle), and
 * ncclCommGetAsyncError reports a system error when FAKE_NCCL_ASYNC_ERROR=1.  The driver entry point
 * is looked up in the libcuda the process has already loaded; without one (CPU-only tests) the
 * all-reduce does nothing.
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#define FAKE_EXPORT __attribute__((visibility("default")))

typedef struct { char internal[128]; } fake_unique_id;
typedef int (*launch_host_fn)(void *stream, void (*fn)(void *), void *user);

static volatile int g_aborted = 0;

/* Sleeps for the given time in slices of 5 ms and returns early once a communicator has been aborted
 * after the all-reduce was CALLED (the real library ends its kernels on abort; the count is taken at the
 * call, not when the stream gets round to running this function, which may be after the abort). */
typedef struct { long ms; int aborted_at_call; } stall_request;
static void stall(void *user) {
    stall_request *request = (stall_request *)user;
    for (long waited = 0; waited < request->ms && g_aborted == request->aborted_at_call; waited += 5) {
        struct timespec nap = {0, 5 * 1000000L};
        nanosleep(&nap, NULL);
    }
    free(request);
}

FAKE_EXPORT int ncclGetUniqueId(fake_unique_id *id) {
    for (int i = 0; i < 128; i++) id->internal[i] = (char)(i ^ 0x5a);
    return 0;
}
FAKE_EXPORT int ncclCommInitRank(void **comm, int world, fake_unique_id id, int rank) {
    (void)world; (void)id; (void)rank;
    *comm = malloc(16);
    return *comm ? 0 : 2;
}
FAKE_EXPORT int ncclCommDestroy(void *comm) { free(comm); return 0; }
FAKE_EXPORT int ncclCommAbort(void *comm) { g_aborted++; free(comm); return 0; }
FAKE_EXPORT int ncclCommGetAsyncError(void *comm, int *result) {
    (void)comm;
    const char *e = getenv("FAKE_NCCL_ASYNC_ERROR");
    *result = (e && e[0] == '1') ? 2 /* ncclSystemError */ : 0;
    return 0;
}
FAKE_EXPORT int ncclGroupStart(void) { return 0; }
FAKE_EXPORT int ncclGroupEnd(void) { return 0; }
FAKE_EXPORT int ncclAllReduce(const void *send, void *recv, size_t count, int dtype, int op, void *comm, void *stream) {
    (void)send; (void)recv; (void)count; (void)dtype; (void)op; (void)comm;
    const char *e = getenv("FAKE_NCCL_STALL_MS");
    long ms = e ? atol(e) : 0;
    if (ms <= 0) return 0;
    void *cuda = dlopen("libcuda.so.1", RTLD_NOW | RTLD_NOLOAD);
    launch_host_fn launch = cuda ? (launch_host_fn)dlsym(cuda, "cuLaunchHostFunc") : NULL;
    if (!launch) return 0;
    stall_request *request = (stall_request *)malloc(sizeof *request);
    if (!request) return 2;
    request->ms = ms; request->aborted_at_call = g_aborted;
    return launch(stream, stall, request) == 0 ? 0 : 1;
}
FAKE_EXPORT int fake_nccl_abort_count(void) { return g_aborted; }
