// Host runtime behind the C ABI: contexts, buffers, prepared executables, the device-resident
// optimizer and the data-parallel communicator.  Handles are tagged structs so a handle of the
// wrong family is rejected instead of being dereferenced as the wrong type (the Metal library
// does the same, modules/backend/metal/macos-arm64/README.md "Status values": 10).
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <time.h>

#include <algorithm>
#include <array>
#include <chrono>
#include <climits>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/synaptik_cuda.h"
#include "kernels.hpp"
#include "lowering.hpp"
#include "program.hpp"

using namespace syn;

namespace {

enum : uint32_t { TAG_CONTEXT = 0x58544353u, TAG_BUFFER = 0x46554253u, TAG_EXECUTABLE = 0x45584553u,
                  TAG_OPTIMIZER = 0x54504f53u, TAG_COMM = 0x4d4f4353u };

struct Optimizer;
struct Comm;

struct Context {
    uint32_t tag = TAG_CONTEXT;
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr, comm_stream = nullptr, copy_stream = nullptr;
    int *error_dev = nullptr;       // device-side error word shared by all kernels of the context
    int *error_host = nullptr;      // pinned mirror
    int gemm_engine = 0;
    int time_steps = 0;
    int fused_planes = 1;
    int gemm_promote = 1;
    int gemm_pair = 1;
    int gemm_dynamic = 1;                   // two-SM products take their tiles from a counter instead of a fixed assignment
    int gemm_slices = 1;                    // split long contractions of epilogue-free GEMMs when that shortens the last wave
    int gemm_chunk = 0;                     // contraction steps per tensor-memory partial sum (0 = default), a multiple of 32
    cudaEvent_t timer_start = nullptr, timer_stop = nullptr;
    cudaEvent_t drained = nullptr;          // recorded behind the error-word copy of a drain; polled when a communicator exists
    int64_t comm_timeout_ms = 30000;        // host-side deadline of every wait that has a collective in front of it
    std::vector<Optimizer *> optimizers;    // a failed drain rolls their unfinished steps back
    std::vector<Comm *> comms;
    std::mutex mutex;
};

struct Buffer {
    uint32_t tag = TAG_BUFFER;
    Context *ctx = nullptr;
    void *ptr = nullptr;
    uint64_t bytes = 0;
    // prefetch ordering (created on first use): `filled` is recorded on the copy stream after a
    // prefetch, `released` on the compute stream after every executable run bound to the buffer
    cudaEvent_t filled = nullptr, released = nullptr;
    bool fill_pending = false, release_recorded = false;
};

// ---- NCCL, bound at run time so the library loads (and inference runs) without it ---------------
struct NcclApi {
    typedef struct { char internal[128]; } UniqueId;
    int (*GetUniqueId)(UniqueId *) = nullptr;
    int (*CommInitRank)(void **, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*CommGetAsyncError)(void *, int *) = nullptr;      // optional: polled while the host waits
    int (*CommAbort)(void *) = nullptr;                     // optional: ends a collective that will never finish
    bool ok = false;
};

NcclApi &nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // An explicit path decides alone (a file that does not load leaves the communicator unavailable,
        // it is not replaced by another copy); otherwise the copy the process already uses, then the
        // loader's own search.
        const char *env = getenv("SYNAPTIK_NCCL_LIBRARY");
        void *h = nullptr;
        if (env && env[0]) h = dlopen(env, RTLD_NOW | RTLD_GLOBAL);
        else {
            h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
            if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
            if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        }
        if (!h) return;
        api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
        api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
        api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
        api.AllReduce = (decltype(api.AllReduce))dlsym(h, "ncclAllReduce");
        api.GroupStart = (decltype(api.GroupStart))dlsym(h, "ncclGroupStart");
        api.GroupEnd = (decltype(api.GroupEnd))dlsym(h, "ncclGroupEnd");
        api.CommGetAsyncError = (decltype(api.CommGetAsyncError))dlsym(h, "ncclCommGetAsyncError");
        api.CommAbort = (decltype(api.CommAbort))dlsym(h, "ncclCommAbort");
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.GroupStart && api.GroupEnd;
    });
    return api;
}

struct Comm {
    uint32_t tag = TAG_COMM;
    Context *ctx = nullptr;
    void *comm = nullptr;
    int world = 1, rank = 0;
    bool dead = false;                      // aborted after a deadline or an asynchronous error: every later use fails
};

struct Planes { float *hi = nullptr, *lo = nullptr; int64_t rows = 0, kp = 0, pitch = 0; int last_run = -1; };

// Identity of an operand's planes: the storage it views and how the plane rows / columns walk it.
// Two program values that view the same storage the same way (a value and PERMUTE of PERMUTE of it)
// share planes; a value and its transpose do not.
typedef std::array<int64_t, 7> PlaneKey;
PlaneKey plane_key(const View &v, int orientation) {
    int r = orientation, c = 1 - orientation;
    return PlaneKey{(int64_t)v.slot, (int64_t)v.index, v.offset, v.shape[r], v.shape[r] == 1 ? 0 : v.strides[r],
                    v.shape[c], v.shape[c] == 1 ? 0 : v.strides[c]};
}

struct StepExec {
    kern::TensorCoreGemm *tc = nullptr;
    int planes_a = -1, planes_b = -1;       // indices into Executable::planes of the MATMUL's two operands
    int orient_a = 0, orient_b = 1;         // which axis of the operand view the plane rows follow
    bool swapped = false;                   // result stored transposed: roles of the operands exchanged
    double *colsum_partials = nullptr;
    float *row_loss = nullptr;
    float *narrow_partials = nullptr;
    int emit_planes = -1;                   // planes this tensor-core step writes from its epilogue
    // what the tensor-core plan was made from, kept so that it can be made again (attach_comm)
    kern::TcOperand tc_p, tc_q;
    int64_t tc_m = 0, tc_n = 0;
    int tc_mode = 0;
    bool tc_plain = false;
};

struct Executable {
    uint32_t tag = TAG_EXECUTABLE;
    Context *ctx = nullptr;
    Program program;
    Plan plan;
    std::vector<void *> scratch;
    void *constants = nullptr;              // 8 bytes per constant slot
    std::vector<Planes> planes;
    std::map<PlaneKey, int> plane_index;
    float *gemm_workspace = nullptr;        // partial products of GEMMs whose contraction is split into slices
    int64_t gemm_workspace_floats = 0;
    int *unit_counters = nullptr;           // one per plan step, zeroed at the start of every run (dynamic tile assignment)
    std::vector<StepExec> exec;
    std::vector<void *> owned;              // every device allocation, for release
    std::vector<uint64_t> feed_bytes, publication_bytes;
    cudaEvent_t start = nullptr, stop = nullptr;
    bool timed = false;
    uint64_t launches = 0;
    int run_counter = 0;
    Comm *comm = nullptr;
    std::vector<char> sync_publication;     // per publication: all-reduce it
    std::vector<cudaEvent_t> ready_events;
    std::vector<cudaEvent_t> step_events;   // two per plan step when the context times steps
    bool steps_timed = false;
    cudaEvent_t comm_done = nullptr;
    bool pending = false;
};

struct Optimizer {
    uint32_t tag = TAG_OPTIMIZER;
    Context *ctx = nullptr;
    int kind = 0;
    double hyper[5] = {0, 0, 0, 0, 0};
    std::vector<Buffer *> params;
    std::vector<uint64_t> counts;
    std::vector<float *> m, v;
    // A step writes candidates into the second set and the host then exchanges the sets (for the
    // parameters: the device pointers of the caller's buffer handles); a failed step is undone by
    // exchanging them back, so what the step read is what is current again.
    std::vector<float *> p_alt, m_alt, v_alt;
    std::vector<float *> acc;               // pending gradient sums, allocated on the first accumulating run
    uint64_t steps = 0;
    uint64_t accumulated_runs = 0;          // runs in the pending sum (TrainingSession.java:593-594)
    bool acc_dirty = false;                 // the pending sums may be non-zero
    bool pending = false;
    // Runs enqueued since the last drain of the context's error word, oldest first, each with the host
    // counters as they were before it.  The kernels of run i carry sequence number i; the device keeps
    // the smallest sequence number that skipped or failed in *failed_dev.
    struct Entry { bool stepped; uint64_t steps, accumulated_runs; bool acc_dirty; };
    std::vector<Entry> journal;
    int *failed_dev = nullptr;
};

template <typename T> T *as(void *h, uint32_t tag) {
    if (!h) return nullptr;
    T *p = reinterpret_cast<T *>(h);
    return p->tag == tag ? p : nullptr;
}

int32_t cuda_status(cudaError_t e, int32_t fallback) {
    if (e == cudaSuccess) return OK;
    if (e == cudaErrorMemoryAllocation) return ALLOCATION_FAILED;
    if (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver || e == cudaErrorInvalidDevice) return NO_DEVICE;
    return fallback;
}

int32_t error_word_status(int word) {
    if (word & kern::ERR_COMM) return COMM_FAILED;
    if (word & kern::ERR_WAIT_TIMEOUT) return TIMEOUT;
    if (word & kern::ERR_LABEL_RANGE) return RANGE_OUT_OF_BOUNDS;
    if (word & kern::ERR_NON_FINITE) return EXECUTION_FAILED;
    return OK;
}

constexpr int kNoFailedSequence = 0x7f7f7f7f;       // what cudaMemset(.., 0x7f, 4) leaves: larger than any sequence number

// Makes the candidate set of an optimizer current, or the previous set current again (the exchange is
// its own inverse).  The parameter pointers live in the caller's buffer handles.
void exchange_sets(Optimizer *o) {
    for (size_t i = 0; i < o->params.size(); i++) {
        void *current = o->params[i]->ptr;
        o->params[i]->ptr = o->p_alt[i];
        o->p_alt[i] = (float *)current;
        if (o->m[i]) std::swap(o->m[i], o->m_alt[i]);
        if (o->v[i]) std::swap(o->v[i], o->v_alt[i]);
    }
}

// After a drain (the compute stream is idle).  A clean drain makes every enqueued step final.  A failed
// one undoes, per optimizer, every run from the first that skipped or failed: those kernels wrote
// candidates at most, so putting the pointers and the host counters back restores parameters, moments,
// pending sums and step count to the bits they had before that run.
void settle_optimizers(Context *ctx, bool failed) {
    for (Optimizer *o : ctx->optimizers) {
        if (o->journal.empty()) continue;
        if (failed) {
            int first = kNoFailedSequence;
            if (cudaMemcpy(&first, o->failed_dev, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); first = 0; }
            cudaMemset(o->failed_dev, 0x7f, sizeof(int));
            if (first >= 0 && first < (int)o->journal.size()) {
                int undone = 0;
                for (size_t i = (size_t)first; i < o->journal.size(); i++) undone += o->journal[i].stepped ? 1 : 0;
                if (undone & 1) exchange_sets(o);
                const Optimizer::Entry &before = o->journal[first];
                o->steps = before.steps; o->accumulated_runs = before.accumulated_runs; o->acc_dirty = before.acc_dirty;
            }
        }
        o->journal.clear();
    }
}

// Waits for `event` (recorded on the compute stream) while a communicator exists: the host polls
// instead of blocking, looks at NCCL's asynchronous error state and gives up after the context's
// comm_timeout_ms.  Giving up marks the context's error word (so that optimizer steps queued behind the
// collective become void), aborts the communicators, which ends their kernels, and then lets the
// streams run dry.  Returns OK or COMM_FAILED with the streams idle either way.
int32_t wait_with_deadline(Context *ctx, cudaEvent_t event) {
    const auto start = std::chrono::steady_clock::now();
    bool failed = false;
    for (uint64_t spin = 0;; spin++) {
        cudaError_t q = cudaEventQuery(event);
        if (q == cudaSuccess) return OK;
        if (q != cudaErrorNotReady) { cudaGetLastError(); return EXECUTION_FAILED; }
        if ((spin & 127u) != 127u) continue;
        for (Comm *c : ctx->comms) {
            int async = 0;
            if (c->dead) continue;          // already given up on: nothing of it is in flight
            if (nccl().CommGetAsyncError && nccl().CommGetAsyncError(c->comm, &async) == 0 && async != 0 && async != 7 /*ncclInProgress*/) failed = true;
        }
        const auto waited = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - start).count();
        if (waited > ctx->comm_timeout_ms * 1000) failed = true;
        if (failed) break;
        if (waited > 5000) {            // a long wait: stop spinning at full speed
            struct timespec nap = {0, 50000};
            nanosleep(&nap, nullptr);
        }
    }
    int word = kern::ERR_COMM;
    if (cudaMemcpyAsync(ctx->error_dev, &word, sizeof(int), cudaMemcpyHostToDevice, ctx->copy_stream) == cudaSuccess) cudaStreamSynchronize(ctx->copy_stream);
    for (Comm *c : ctx->comms) {
        if (!c->dead && nccl().CommAbort) { nccl().CommAbort(c->comm); c->comm = nullptr; }
        c->dead = true;
    }
    cudaStreamSynchronize(ctx->comm_stream);
    cudaStreamSynchronize(ctx->stream);
    cudaGetLastError();
    return COMM_FAILED;
}

// Reads and clears the device error word; the stream is synchronised on return.  A failure undoes the
// optimizer steps that did not take place (settle_optimizers).
int32_t drain_errors(Context *ctx) {
    cudaError_t e = cudaMemcpyAsync(ctx->error_host, ctx->error_dev, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(ctx->error_dev, 0, sizeof(int), ctx->stream);
    int32_t status = OK;
    if (e == cudaSuccess && !ctx->comms.empty()) {
        if (!ctx->drained) e = cudaEventCreateWithFlags(&ctx->drained, cudaEventDisableTiming);
        if (e == cudaSuccess) e = cudaEventRecord(ctx->drained, ctx->stream);
        if (e == cudaSuccess) status = wait_with_deadline(ctx, ctx->drained);
    } else if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) { cudaGetLastError(); status = EXECUTION_FAILED; }
    if (status == OK) status = error_word_status(*ctx->error_host);
    settle_optimizers(ctx, status != OK);
    return status;
}

struct DeviceGuard {
    int previous = -1;
    explicit DeviceGuard(int device) { cudaGetDevice(&previous); if (previous != device) cudaSetDevice(device); else previous = -1; }
    ~DeviceGuard() { if (previous >= 0) cudaSetDevice(previous); }
};

void bswap_copy(uint8_t *dst, const uint8_t *src, uint64_t bytes, uint32_t width) {
    if (width == 1) { memcpy(dst, src, bytes); return; }
    for (uint64_t i = 0; i + width <= bytes; i += width)
        for (uint32_t b = 0; b < width; b++) dst[i + b] = src[i + width - 1 - b];
}

kern::Index4 index4(const std::vector<int64_t> &shape, const std::vector<int64_t> *sa, const std::vector<int64_t> *sb,
                    const std::vector<int64_t> *sc, const std::vector<int64_t> *shape_a = nullptr,
                    const std::vector<int64_t> *shape_b = nullptr, const std::vector<int64_t> *shape_c = nullptr) {
    // right-aligns every operand against `shape`; broadcast axes (extent 1 against a larger one) get stride 0
    kern::Index4 ix;
    size_t r = shape.size();
    for (int d = 0; d < 4; d++) { ix.shape[d] = 1; ix.sa[d] = ix.sb[d] = ix.sc[d] = 0; }
    auto fill = [&](int64_t *dst, const std::vector<int64_t> *strides, const std::vector<int64_t> *oshape) {
        if (!strides) return;
        size_t orank = strides->size();
        for (size_t d = 0; d < orank; d++) {
            size_t target = 4 - orank + d;
            int64_t extent = oshape ? (*oshape)[d] : shape[r - orank + d];
            dst[target] = extent == 1 ? 0 : (*strides)[d];
        }
    };
    for (size_t d = 0; d < r; d++) ix.shape[4 - r + d] = shape[d];
    fill(ix.sa, sa, shape_a); fill(ix.sb, sb, shape_b); fill(ix.sc, sc, shape_c);
    return ix;
}

struct Binding {
    std::vector<Buffer *> feeds, publications;
};

uint64_t view_span_bytes(const View &v) {
    int64_t last = v.offset;
    for (size_t d = 0; d < v.shape.size(); d++) { if (v.shape[d] == 0) return 0; last += (v.shape[d] - 1) * v.strides[d]; }
    return (uint64_t)(last + 1) * dtype_bytes(v.dtype);
}

int32_t prepare_executable(Executable *x) {
    Context *ctx = x->ctx;
    const Plan &plan = x->plan;
    auto alloc = [&](uint64_t bytes, void **out) -> bool {
        void *p = nullptr;
        if (cudaMalloc(&p, bytes ? bytes : 4) != cudaSuccess) { cudaGetLastError(); return false; }
        x->owned.push_back(p);
        *out = p;
        return true;
    };
    for (int64_t bytes : plan.scratch_bytes) { void *p; if (!alloc((uint64_t)bytes, &p)) return ALLOCATION_FAILED; x->scratch.push_back(p); }
    if (!plan.constant_values.empty()) {
        std::vector<uint64_t> host(plan.constant_values.size(), 0);
        for (size_t i = 0; i < host.size(); i++) {
            const Value &v = x->program.values[plan.constant_values[i]];
            if (v.dtype == DType::F32) { float f = (float)v.constant_f64(); memcpy(&host[i], &f, 4); }
            else if (v.dtype == DType::I32) { int32_t q = (int32_t)v.constant_i64(); memcpy(&host[i], &q, 4); }
            else if (v.dtype == DType::I64) { int64_t q = v.constant_i64(); memcpy(&host[i], &q, 8); }
            else { uint8_t q = v.constant_i64() != 0; memcpy(&host[i], &q, 1); }
        }
        if (!alloc(host.size() * 8, &x->constants)) return ALLOCATION_FAILED;
        if (cudaMemcpy(x->constants, host.data(), host.size() * 8, cudaMemcpyHostToDevice) != cudaSuccess) return COPY_FAILED;
    }
    x->feed_bytes.assign(x->program.feeds.size(), 0);
    x->publication_bytes.assign(x->program.publications.size(), 0);
    for (const View &v : plan.views) {
        if (v.index < 0) continue;
        if (v.slot == SlotKind::FEED) x->feed_bytes[v.index] = std::max(x->feed_bytes[v.index], view_span_bytes(v));
        if (v.slot == SlotKind::PUBLICATION) x->publication_bytes[v.index] = std::max(x->publication_bytes[v.index], view_span_bytes(v));
    }
    x->exec.resize(plan.steps.size());
    int64_t workspace_floats = 0;               // one workspace serves every sliced GEMM: the steps run in stream order
    auto planes_for = [&](int value, int orientation, int64_t rows, int64_t k) -> int {
        PlaneKey key = plane_key(plan.views[value], orientation);
        auto it = x->plane_index.find(key);
        if (it != x->plane_index.end()) return it->second;
        Planes p;
        p.rows = rows; p.kp = kern::padded_k(k); p.pitch = kern::plane_pitch(p.kp);
        void *hi, *lo;
        if (!alloc((uint64_t)rows * p.pitch * 4, &hi) || !alloc((uint64_t)rows * p.pitch * 4, &lo)) return -1;
        // padding columns are zero from the start: the pass that fills planes beside the column sums
        // only writes the real columns
        if (cudaMemsetAsync(hi, 0, (uint64_t)rows * p.pitch * 4, ctx->stream) != cudaSuccess
            || cudaMemsetAsync(lo, 0, (uint64_t)rows * p.pitch * 4, ctx->stream) != cudaSuccess) return -1;
        p.hi = (float *)hi; p.lo = (float *)lo;
        x->planes.push_back(p);
        x->plane_index[key] = (int)x->planes.size() - 1;
        return (int)x->planes.size() - 1;
    };
    for (size_t i = 0; i < plan.steps.size(); i++) {
        const Step &st = plan.steps[i];
        StepExec &se = x->exec[i];
        if (st.kind == StepKind::GEMM && st.engine == GemmEngine::TENSOR_CORE && !dtype_low(plan.views[st.a].dtype)) {
            const View &c = plan.views[st.out];
            se.swapped = c.strides[0] == 1 && c.shape[0] != 1 && c.strides[1] != 1;
            // Plane rows follow the axis of the operand view that is NOT contiguous, so every split is a
            // row split; an operand whose contraction axis is the strided one is handed to the kernel as
            // MN-major planes ([k, rows]) instead of being transposed.  Orientation 0: plane rows follow
            // axis 0 of the view, 1: axis 1.  A = [m, k] is K-major at orientation 0, B = [k, n] at 1.
            const View &va = plan.views[st.a], &vb = plan.views[st.b];
            se.orient_a = (va.strides[1] == 1 || va.shape[1] == 1) ? 0 : 1;
            se.orient_b = (vb.strides[0] == 1 || vb.shape[0] == 1) ? 1 : 0;
            if ((se.orient_a == 1 && va.strides[0] != 1) || (se.orient_b == 0 && vb.strides[1] != 1)) return UNSUPPORTED_SHAPE;
            se.planes_a = se.orient_a == 0 ? planes_for(st.a, 0, st.m, st.k) : planes_for(st.a, 1, st.k, st.m);
            se.planes_b = se.orient_b == 1 ? planes_for(st.b, 1, st.n, st.k) : planes_for(st.b, 0, st.k, st.n);
            if (se.planes_a < 0 || se.planes_b < 0) return ALLOCATION_FAILED;
            const Planes &A = x->planes[se.planes_a], &B = x->planes[se.planes_b];
            kern::TcOperand oa, ob;
            oa.hi = A.hi; oa.lo = A.lo; oa.pitch = A.pitch; oa.mn_major = se.orient_a == 1;
            ob.hi = B.hi; ob.lo = B.lo; ob.pitch = B.pitch; ob.mn_major = se.orient_b == 0;
            int status = OK;
            const bool plain = st.bias < 0 && st.mask < 0 && !st.relu && !st.act && st.out2 < 0;
            const int mode = ctx->gemm_promote | (ctx->gemm_pair << 1) | ((plain && ctx->gemm_slices) ? 4 : 0) | ((plain && ctx->gemm_slices == 2) ? 8 : 0) | ((ctx->gemm_chunk / 32) << 8);
            se.tc_p = se.swapped ? ob : oa; se.tc_q = se.swapped ? oa : ob;
            se.tc_m = se.swapped ? st.n : st.m; se.tc_n = se.swapped ? st.m : st.n;
            se.tc_mode = mode; se.tc_plain = plain;
            se.tc = kern::tc_gemm_prepare(se.tc_p, se.tc_q, se.tc_m, se.tc_n, st.k, ctx->sm_count, mode, &status);
            if (se.tc) workspace_floats = std::max(workspace_floats, kern::tc_gemm_workspace_floats(se.tc));
            if (!se.tc) return status;
        } else if (st.kind == StepKind::GEMM && st.engine == GemmEngine::NARROW_REDUCE) {
            void *p; if (!alloc((uint64_t)kern::narrow_reduce_partial_floats(st.m, st.n, st.k) * 4, &p)) return ALLOCATION_FAILED;
            se.narrow_partials = (float *)p;
        } else if (st.kind == StepKind::COLSUM) {
            void *p; if (!alloc((uint64_t)kern::colsum_partial_count(st.m, st.n) * 8, &p)) return ALLOCATION_FAILED;
            se.colsum_partials = (double *)p;
        } else if (st.kind == StepKind::MSE && st.scalar_bits != 0 && kern::mse_partial_count(st.m) > 0) {
            void *p; if (!alloc((uint64_t)kern::mse_partial_count(st.m) * 8, &p)) return ALLOCATION_FAILED;
            se.colsum_partials = (double *)p;       // the same kind of scratch: binary64 partial sums
        } else if (st.kind == StepKind::CROSS_ENTROPY || st.kind == StepKind::DENSE_CROSS_ENTROPY) {
            void *p; if (!alloc((uint64_t)(st.m + 4) * 4, &p)) return ALLOCATION_FAILED;     // row losses, then one cell for the count of rows left
            se.row_loss = (float *)p;
        }
    }
    if (workspace_floats > 0) {
        void *p; if (!alloc((uint64_t)workspace_floats * 4, &p)) return ALLOCATION_FAILED;
        x->gemm_workspace = (float *)p;
        x->gemm_workspace_floats = workspace_floats;
    }
    if (ctx->gemm_dynamic) {
        void *p; if (!alloc((uint64_t)plan.steps.size() * 4, &p)) return ALLOCATION_FAILED;
        x->unit_counters = (int *)p;
    }
    // a tensor-core GEMM whose dense result is later read as a GEMM operand writes that operand's
    // planes itself, which removes the separate split pass
    for (size_t i = 0; i < plan.steps.size(); i++) {
        const Step &st = plan.steps[i];
        StepExec &se = x->exec[i];
        // fused_planes 1 (default): where it pays.  That is every two-SM product with the staged write-out
        // (measured on the training step, cycle counts of all launches: 79.3 M clocks per step against 81.7 with
        // separate split passes) and, on the other kernels, one-accumulator products with a long main loop
        // (direct stores: a K = 784 producer doubled in time, K = 4096 producers gained; with FP32 promotion
        // the extra direct stores bought nothing).  2: every producer with K >= 2048; 3: every producer.
        // A product whose contraction is split into slices has no epilogue of its own: its planes are
        // written by the ordinary split pass.
        if (st.kind != StepKind::GEMM || st.engine != GemmEngine::TENSOR_CORE || !se.tc || se.swapped || !ctx->fused_planes) continue;
        if (ctx->fused_planes == 1 && !kern::tc_gemm_staged_shape(se.tc) && (ctx->gemm_promote || st.k < 2048)) continue;
        if (ctx->fused_planes == 2 && st.k < 2048) continue;
        if (kern::tc_gemm_launches(se.tc) > 1) continue;
        const View &u = plan.views[st.out2 >= 0 ? st.out2 : st.out];
        if (u.shape.size() != 2 || !u.dense()) continue;
        auto normal = x->plane_index.find(plane_key(u, 0));
        if (normal != x->plane_index.end()) se.emit_planes = normal->second;
    }
    if (cudaEventCreate(&x->start) != cudaSuccess || cudaEventCreate(&x->stop) != cudaSuccess) return INTERNAL_ERROR;
    x->sync_publication.assign(x->program.publications.size(), 0);
    return OK;
}

void release_executable(Executable *x) {
    DeviceGuard guard(x->ctx->device);
    cudaStreamSynchronize(x->ctx->stream);
    cudaStreamSynchronize(x->ctx->comm_stream);
    for (StepExec &se : x->exec) if (se.tc) kern::tc_gemm_release(se.tc);
    for (void *p : x->owned) cudaFree(p);
    if (x->start) cudaEventDestroy(x->start);
    if (x->stop) cudaEventDestroy(x->stop);
    if (x->comm_done) cudaEventDestroy(x->comm_done);
    for (cudaEvent_t e : x->ready_events) cudaEventDestroy(e);
    for (cudaEvent_t e : x->step_events) cudaEventDestroy(e);
    x->tag = 0;
    delete x;
}

#define LAUNCH(expr) do { cudaError_t e_ = (expr); x->launches++; if (e_ != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; } } while (0)

int32_t enqueue_executable(Executable *x, const Binding &bind) {
    Context *ctx = x->ctx;
    const Plan &plan = x->plan;
    cudaStream_t s = ctx->stream;
    auto base = [&](const View &v) -> uint8_t * {
        switch (v.slot) {
            case SlotKind::FEED: return (uint8_t *)bind.feeds[v.index]->ptr;
            case SlotKind::PUBLICATION: return (uint8_t *)bind.publications[v.index]->ptr;
            case SlotKind::SCRATCH: return (uint8_t *)x->scratch[v.index];
            case SlotKind::CONSTANT: return (uint8_t *)x->constants + 8 * (size_t)v.index;
        }
        return nullptr;
    };
    auto ptr = [&](int value) -> void * {
        if (value < 0) return nullptr;
        const View &v = plan.views[value];
        return base(v) + (v.slot == SlotKind::CONSTANT ? 0 : v.offset * dtype_bytes(v.dtype));
    };
    x->launches = 0;
    x->run_counter++;
    if (x->unit_counters && cudaMemsetAsync(x->unit_counters, 0, plan.steps.size() * 4, s) != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
    // buffers filled by a prefetch on the copy stream: this run (and, by stream order, every later
    // one) starts after the copy
    for (const std::vector<Buffer *> *group : {&bind.feeds, &bind.publications})
        for (Buffer *b : *group)
            if (b->fill_pending) { cudaStreamWaitEvent(s, b->filled, 0); b->fill_pending = false; }
    cudaEventRecord(x->start, s);
    int ready_cursor = 0;
    const bool time_steps = ctx->time_steps != 0;
    if (time_steps && x->step_events.size() < 2 * plan.steps.size()) {
        while (x->step_events.size() < 2 * plan.steps.size()) {
            cudaEvent_t e; if (cudaEventCreate(&e) != cudaSuccess) return INTERNAL_ERROR;
            x->step_events.push_back(e);
        }
    }
    x->steps_timed = time_steps;
    for (size_t i = 0; i < plan.steps.size(); i++) {
        const Step &st = plan.steps[i];
        StepExec &se = x->exec[i];
        const bool tc_step = st.kind == StepKind::GEMM && st.engine == GemmEngine::TENSOR_CORE && se.tc;
        if (time_steps && !tc_step) cudaEventRecord(x->step_events[2 * i], s);
        switch (st.kind) {
            case StepKind::GEMM: {
                const View &a = plan.views[st.a], &b = plan.views[st.b], &c = plan.views[st.out];
                kern::GemmEpilogue ep;
                ep.bias = (const float *)ptr(st.bias);
                ep.gate = (const float *)ptr(st.mask);
                ep.act = st.relu ? (int)Op::RELU : st.act;        // with a second output: out = z, second = act(z)
                ep.second = (float *)ptr(st.out2);
                if (dtype_low(a.dtype)) {
                    // 16-bit storage: tensor cores straight from the operands, or the exact chain
                    const int kind = a.dtype == DType::BF16 ? 1 : 2;
                    const int act = st.relu ? (int)Op::RELU : st.act;
                    cudaError_t le = cudaErrorInvalidValue;
                    if (st.engine == GemmEngine::TENSOR_CORE)
                        le = kern::low_gemm_launch(s, kind, ctx->sm_count, st.m, st.n, st.k, ptr(st.a), a.strides[0], ptr(st.b), b.strides[1],
                                                   ptr(st.out), c.strides[0], ptr(st.bias), act, ptr(st.out2), ctx->gemm_chunk, ctx->error_dev);
                    if (le != cudaSuccess) {        // a misaligned binding: the exact kernel takes every shape and alignment
                        cudaGetLastError();
                        le = kern::gemm_exact_low(s, kind, st.m, st.n, st.k, ptr(st.a), a.strides[0], a.strides[1], ptr(st.b), b.strides[0], b.strides[1],
                                                  ptr(st.out), c.strides[0], c.strides[1], ptr(st.bias), act, ptr(st.out2));
                    }
                    LAUNCH(le);
                    break;
                }
                cudaError_t narrow = cudaErrorInvalidValue;
                if (st.engine == GemmEngine::NARROW_OUT)
                    narrow = kern::gemm_narrow_out(s, ctx->sm_count, st.m, st.n, st.k, (const float *)ptr(st.a), a.strides[0], (const float *)ptr(st.b),
                                                   b.strides[1], ep.bias, st.relu ? 1 : 0, (float *)ptr(st.out), c.strides[0], c.strides[1]);
                else if (st.engine == GemmEngine::NARROW_INNER)
                    narrow = kern::gemm_narrow_inner(s, st.m, st.n, st.k, (const float *)ptr(st.a), a.strides[0], (const float *)ptr(st.b),
                                                     b.strides[0], ep.gate, (float *)ptr(st.out), c.strides[0]);
                else if (st.engine == GemmEngine::NARROW_REDUCE)
                    narrow = kern::gemm_narrow_reduce(s, st.m, st.n, st.k, (const float *)ptr(st.a), a.strides[1], (const float *)ptr(st.b),
                                                      b.strides[0], se.narrow_partials, (float *)ptr(st.out), c.strides[0], c.strides[1]);
                if (st.engine != GemmEngine::TENSOR_CORE && st.engine != GemmEngine::EXACT_SIMT && narrow == cudaSuccess) {
                    x->launches += st.engine == GemmEngine::NARROW_REDUCE ? 2 : 1;
                } else if (st.engine != GemmEngine::TENSOR_CORE) {
                    // the exact kernel takes every shape and alignment (and is what a misaligned view falls back to)
                    cudaGetLastError();
                    LAUNCH(kern::gemm_exact(s, st.m, st.n, st.k, (const float *)ptr(st.a), a.strides[0], a.strides[1],
                                            (const float *)ptr(st.b), b.strides[0], b.strides[1],
                                            (float *)ptr(st.out), c.strides[0], c.strides[1], ep));
                } else {
                    // operands are immutable within a run: split each (value, orientation) once per run
                    auto split = [&](int value, int orientation, int index) -> int32_t {
                        Planes &pl = x->planes[index];
                        if (pl.last_run == x->run_counter) return OK;
                        const View &v = plan.views[value];
                        LAUNCH(kern::split_planes(s, (const float *)ptr(value), pl.rows, v.shape[1 - orientation], v.strides[orientation],
                                                  pl.hi, pl.lo, pl.pitch));
                        pl.last_run = x->run_counter;
                        return OK;
                    };
                    int32_t r1 = split(st.a, se.orient_a, se.planes_a); if (r1 != OK) return r1;
                    int32_t r2 = split(st.b, se.orient_b, se.planes_b); if (r2 != OK) return r2;
                    int64_t ldd = se.swapped ? c.strides[1] : c.strides[0];
                    if (se.emit_planes >= 0) {
                        Planes &pl = x->planes[se.emit_planes];
                        ep.plane_hi = pl.hi; ep.plane_lo = pl.lo; ep.plane_ld = pl.pitch; pl.last_run = x->run_counter;
                    }
                    if (time_steps) cudaEventRecord(x->step_events[2 * i], s);
                    LAUNCH(kern::tc_gemm_launch(s, se.tc, (float *)ptr(st.out), ldd, ep, x->gemm_workspace,
                                                x->unit_counters ? x->unit_counters + i : nullptr, ctx->error_dev));
                    x->launches += kern::tc_gemm_launches(se.tc) - 1;
                }
                break;
            }
            case StepKind::BINARY: {
                const View &a = plan.views[st.a], &b = plan.views[st.b], &o = plan.views[st.out];
                kern::Index4 ix = index4(o.shape, &a.strides, &b.strides, nullptr, &a.shape, &b.shape, nullptr);
                int64_t total = 1; for (auto d : o.shape) total *= d;
                if (dtype_low(a.dtype)) LAUNCH(kern::binary_low(s, a.dtype == DType::BF16 ? 1 : 2, st.op, ptr(st.a), ptr(st.b), ptr(st.out), ix, total));
                else if (a.dtype == DType::F32) LAUNCH(kern::binary(s, st.op, (const float *)ptr(st.a), (const float *)ptr(st.b), ptr(st.out), ix, total));
                else LAUNCH(kern::binary_int(s, st.op, a.dtype, ptr(st.a), ptr(st.b), ptr(st.out), ix, total));
                break;
            }
            case StepKind::WHERE: {
                const View &a = plan.views[st.a], &b = plan.views[st.b], &c = plan.views[st.c], &o = plan.views[st.out];
                kern::Index4 ix = index4(o.shape, &a.strides, &b.strides, &c.strides, &a.shape, &b.shape, &c.shape);
                int64_t total = 1; for (auto d : o.shape) total *= d;
                LAUNCH(kern::where(s, (const uint8_t *)ptr(st.a), (const float *)ptr(st.b), (const float *)ptr(st.c), (float *)ptr(st.out), ix, total));
                break;
            }
            case StepKind::SCALAR: case StepKind::UNARY: {
                const View &a = plan.views[st.a], &o = plan.views[st.out];
                int64_t total = 1; for (auto d : o.shape) total *= d;
                const void *src = ptr(st.a);
                if (!a.dense()) return UNSUPPORTED_SHAPE;
                if (st.kind == StepKind::SCALAR) LAUNCH(kern::scalar_op(s, st.op, a.dtype, src, ptr(st.out), st.scalar_bits, total));
                else if (dtype_low(a.dtype)) LAUNCH(kern::unary_low(s, a.dtype == DType::BF16 ? 1 : 2, st.op, src, ptr(st.out), total));
                else LAUNCH(kern::unary(s, st.op, (const float *)src, ptr(st.out), total));
                break;
            }
            case StepKind::ONE_HOT:
                LAUNCH(kern::one_hot(s, plan.views[st.a].dtype, ptr(st.a), (uint8_t *)ptr(st.out), st.m, st.n));
                break;
            case StepKind::COPY: {
                const View &a = plan.views[st.a], &o = plan.views[st.out];
                kern::Index4 ix = index4(o.shape, &a.strides, nullptr, nullptr, &a.shape);
                int64_t total = 1; for (auto d : o.shape) total *= d;
                LAUNCH(kern::copy_strided(s, dtype_bytes(a.dtype), ptr(st.a), ptr(st.out), ix, total));
                break;
            }
            case StepKind::ROW_REDUCE:
                LAUNCH(kern::row_reduce(s, st.op, (const float *)ptr(st.a), (float *)ptr(st.out), st.m, st.n));
                break;
            case StepKind::FULL_SUM: {
                const View &a = plan.views[st.a];
                kern::Index4 ix = index4(a.shape, &a.strides, nullptr, nullptr, &a.shape);
                LAUNCH(kern::full_sum(s, (const float *)ptr(st.a), ix, st.m, (float *)ptr(st.out)));
                break;
            }
            case StepKind::COLSUM: {
                // a gradient that tensor-core products read as row planes is split in the same pass
                float *hi = nullptr, *lo = nullptr; int64_t pitch = 0;
                const View &v = plan.views[st.a];
                if (v.shape.size() == 2 && v.dense()) {
                    auto it = x->plane_index.find(plane_key(v, 0));
                    if (it != x->plane_index.end()) {
                        Planes &pl = x->planes[it->second];
                        if (pl.last_run != x->run_counter && pl.rows == st.m && kern::colsum_can_split((const float *)ptr(st.a), st.n, pl.pitch)) {
                            hi = pl.hi; lo = pl.lo; pitch = pl.pitch; pl.last_run = x->run_counter;
                        }
                    }
                }
                LAUNCH(kern::colsum(s, (const float *)ptr(st.a), st.m, st.n, se.colsum_partials, (float *)ptr(st.out), hi, lo, pitch));
                x->launches++;
                break;
            }
            case StepKind::SOFTMAX:
                LAUNCH(kern::softmax_rows(s, (const float *)ptr(st.a), (float *)ptr(st.out), st.m, st.n, st.scalar_bits == 1));
                break;
            case StepKind::CROSS_ENTROPY: {
                // reduction of the forward loss node: NONE publishes the row losses themselves
                const int reduction = (int)st.scalar_bits;
                const bool per_row = reduction == 0 && st.out >= 0;
                LAUNCH(kern::cross_entropy(s, (const float *)ptr(st.a), plan.views[st.b].dtype, ptr(st.b), (const float *)ptr(st.c), st.m, st.n,
                                           per_row ? (float *)ptr(st.out) : se.row_loss, per_row ? nullptr : (float *)ptr(st.out),
                                           (float *)ptr(st.out2), (int64_t *)ptr(st.out3), ctx->error_dev, reduction == 2,
                                           st.has_ignore ? 1 : 0, st.ignore, st.scale_mode, se.row_loss + st.m));
                if (st.has_ignore && st.out2 >= 0 && st.scale_mode == 0) x->launches++;
                if (st.out >= 0 && !per_row) x->launches++;
                break;
            }
            case StepKind::DENSE_CROSS_ENTROPY: {
                const int reduction = (int)st.scalar_bits;
                const bool per_row = reduction == 0;
                LAUNCH(kern::dense_cross_entropy(s, (const float *)ptr(st.a), (const float *)ptr(st.b), st.m, st.n,
                                                 per_row ? (float *)ptr(st.out) : se.row_loss, per_row ? nullptr : (float *)ptr(st.out), reduction == 2));
                if (!per_row) x->launches++;
                break;
            }
            case StepKind::SOFTMAX_BACKWARD:
                LAUNCH(kern::softmax_backward_rows(s, (const float *)ptr(st.a), (const float *)ptr(st.b), (float *)ptr(st.out), st.m, st.n, st.scalar_bits == 1));
                break;
            case StepKind::DENSE_CE_BACKWARD:
                LAUNCH(kern::dense_cross_entropy_backward(s, (const float *)ptr(st.a), (const float *)ptr(st.b), (const float *)ptr(st.c), st.m, st.n,
                                                          (float *)ptr(st.out), st.scale_mode));
                break;
            case StepKind::MSE:
                LAUNCH(kern::mse(s, (int)st.scalar_bits, (const float *)ptr(st.a), (const float *)ptr(st.b), st.m, (float *)ptr(st.out), se.colsum_partials));
                if (se.colsum_partials && st.scalar_bits != 0) x->launches++;
                break;
            case StepKind::ARG_MAX:
                if (dtype_low(plan.views[st.a].dtype)) LAUNCH(kern::argmax_rows_low(s, plan.views[st.a].dtype == DType::BF16 ? 1 : 2, ptr(st.a), (int64_t *)ptr(st.out), st.m, st.n));
                else LAUNCH(kern::argmax_rows(s, (const float *)ptr(st.a), (int64_t *)ptr(st.out), st.m, st.n));
                break;
            case StepKind::RELU_BACKWARD: {
                int64_t total = 1; for (auto d : plan.views[st.out].shape) total *= d;
                LAUNCH(kern::relu_backward(s, (const float *)ptr(st.a), (const float *)ptr(st.b), (float *)ptr(st.out), total));
                break;
            }
        }
        if (time_steps) cudaEventRecord(x->step_events[2 * i + 1], s);
        // gradients that are final go to the communication stream at once, so their all-reduce
        // overlaps the rest of the backward pass
        if (x->comm) for (int j : st.ready_publications) if (x->sync_publication[j]) {
            if (ready_cursor >= (int)x->ready_events.size()) {
                cudaEvent_t e; if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return INTERNAL_ERROR;
                x->ready_events.push_back(e);
            }
            cudaEvent_t ev = x->ready_events[ready_cursor++];
            cudaEventRecord(ev, s);
            cudaStreamWaitEvent(ctx->comm_stream, ev, 0);
            Buffer *buf = bind.publications[j];
            uint64_t count = x->publication_bytes[j] / 4;
            if (x->comm->dead || nccl().AllReduce(buf->ptr, buf->ptr, count, /*ncclFloat32*/ 7, /*ncclSum*/ 0, x->comm->comm, ctx->comm_stream) != 0) return COMM_FAILED;
        }
    }
    if (x->comm && ready_cursor > 0) {
        if (!x->comm_done && cudaEventCreateWithFlags(&x->comm_done, cudaEventDisableTiming) != cudaSuccess) return INTERNAL_ERROR;
        cudaEventRecord(x->comm_done, ctx->comm_stream);
        cudaStreamWaitEvent(s, x->comm_done, 0);
    }
    cudaEventRecord(x->stop, s);
    // a later prefetch into one of these buffers has to wait for this run
    for (const std::vector<Buffer *> *group : {&bind.feeds, &bind.publications})
        for (Buffer *b : *group)
            if (b->released) { cudaEventRecord(b->released, s); b->release_recorded = true; }
    x->timed = true;
    x->pending = true;
    return OK;
}

int32_t bind_buffers(Executable *x, int32_t nin, void *const *in, int32_t nout, void *const *out, Binding &bind) {
    if (nin != (int32_t)x->program.feeds.size() || nout != (int32_t)x->program.publications.size()) return INVALID_ARGUMENT;
    if ((nin && !in) || (nout && !out)) return INVALID_ARGUMENT;
    for (int i = 0; i < nin; i++) {
        Buffer *b = as<Buffer>(in[i], TAG_BUFFER);
        if (!b) return INVALID_ARGUMENT;
        if (b->ctx != x->ctx || b->bytes < x->feed_bytes[i]) return INCOMPATIBLE_RESOURCE;
        bind.feeds.push_back(b);
    }
    for (int i = 0; i < nout; i++) {
        Buffer *b = as<Buffer>(out[i], TAG_BUFFER);
        if (!b) return INVALID_ARGUMENT;
        if (b->ctx != x->ctx || b->bytes < x->publication_bytes[i]) return INCOMPATIBLE_RESOURCE;
        for (Buffer *f : bind.feeds) if (f == b) return INCOMPATIBLE_RESOURCE;             // an input aliases an output
        for (Buffer *p : bind.publications) if (p == b) return INCOMPATIBLE_RESOURCE;      // two outputs alias
        bind.publications.push_back(b);
    }
    return OK;
}

int32_t build_program(const uint8_t *program, uint32_t bytes, int gemm_engine, Program &g, Plan &plan) {
    std::string message;
    Status s = parse_program(program, bytes, g, message);
    if (s != OK) return s;
    LoweringOptions options;
    options.gemm_engine = gemm_engine;
    return lower_program(g, options, plan, message);
}

}  // namespace

extern "C" {

uint32_t synaptik_cuda_abi_version(void) { return SYNAPTIK_CUDA_ABI_VERSION; }

int32_t synaptik_cuda_context_create(int32_t device_ordinal, void **out_context) {
    if (!out_context) return INVALID_ARGUMENT;
    *out_context = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) { cudaGetLastError(); return NO_DEVICE; }
    if (device_ordinal < 0 || device_ordinal >= count) return INVALID_ARGUMENT;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device_ordinal) != cudaSuccess) { cudaGetLastError(); return NO_DEVICE; }
    if (prop.major != 10) return NO_DEVICE;         // kernels are built for sm_100a only; there is no other path
    DeviceGuard guard(device_ordinal);
    Context *ctx = new Context();
    ctx->device = device_ordinal;
    ctx->sm_count = prop.multiProcessorCount;
    if (const char *e = getenv("SYNAPTIK_CUDA_GEMM_PAIR")) ctx->gemm_pair = atoi(e) != 0;      // test hook for the default
    // The communication stream gets the highest priority and the compute stream the lowest: an
    // all-reduce that becomes ready while a persistent GEMM grid is also waiting for SMs goes first and
    // takes its few SMs, so it overlaps the GEMM.  The other way round (measured on 4 GPUs) the GEMM
    // takes every SM, the collective waits for the whole GEMM, and the all-reduces pile up behind the
    // backward pass: 15.5 ms per step instead of 14.0.
    int least = 0, greatest = 0;
    cudaDeviceGetStreamPriorityRange(&least, &greatest);
    int compute_priority = least, comm_priority = greatest;
    if (const char *e = getenv("SYNAPTIK_CUDA_STREAM_PRIORITY")) {      // test hook: 0 = no priorities, 1 = compute first
        if (atoi(e) == 0) compute_priority = comm_priority = 0;
        else if (atoi(e) == 1) { compute_priority = greatest; comm_priority = least; }
    }
    if (cudaStreamCreateWithPriority(&ctx->stream, cudaStreamNonBlocking, compute_priority) != cudaSuccess
        || cudaStreamCreateWithPriority(&ctx->comm_stream, cudaStreamNonBlocking, comm_priority) != cudaSuccess
        || cudaStreamCreateWithFlags(&ctx->copy_stream, cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); delete ctx; return NO_STREAM; }
    if (cudaMalloc(&ctx->error_dev, sizeof(int)) != cudaSuccess || cudaMallocHost(&ctx->error_host, sizeof(int)) != cudaSuccess
        || cudaMemset(ctx->error_dev, 0, sizeof(int)) != cudaSuccess) { cudaGetLastError(); delete ctx; return ALLOCATION_FAILED; }
    *out_context = ctx;
    return OK;
}

int32_t synaptik_cuda_context_release(void *context) {
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx) return INVALID_ARGUMENT;
    DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaStreamSynchronize(ctx->comm_stream);
    cudaStreamDestroy(ctx->stream);
    cudaStreamDestroy(ctx->comm_stream);
    cudaStreamDestroy(ctx->copy_stream);
    cudaFree(ctx->error_dev);
    cudaFreeHost(ctx->error_host);
    if (ctx->timer_start) cudaEventDestroy(ctx->timer_start);
    if (ctx->timer_stop) cudaEventDestroy(ctx->timer_stop);
    if (ctx->drained) cudaEventDestroy(ctx->drained);
    ctx->tag = 0;
    delete ctx;
    return OK;
}

int32_t synaptik_cuda_context_set_option(void *context, const char *name, int64_t value) {
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx || !name) return INVALID_ARGUMENT;
    if (!strcmp(name, "gemm_engine")) { if (value < 0 || value > 2) return INVALID_ARGUMENT; ctx->gemm_engine = (int)value; return OK; }
    if (!strcmp(name, "gemm_dynamic")) { if (value < 0 || value > 1) return INVALID_ARGUMENT; ctx->gemm_dynamic = (int)value; return OK; }
    if (!strcmp(name, "gemm_slices")) { if (value < 0 || value > 2) return INVALID_ARGUMENT; ctx->gemm_slices = (int)value; return OK; }
    if (!strcmp(name, "gemm_pair")) { if (value < 0 || value > 1) return INVALID_ARGUMENT; ctx->gemm_pair = (int)value; return OK; }
    if (!strcmp(name, "gemm_chunk")) { if (value < 0 || value > 4096 || value % 32) return INVALID_ARGUMENT; ctx->gemm_chunk = (int)value; return OK; }
    if (!strcmp(name, "gemm_promote")) { if (value < 0 || value > 1) return INVALID_ARGUMENT; ctx->gemm_promote = (int)value; return OK; }
    if (!strcmp(name, "fused_planes")) { if (value < 0 || value > 3) return INVALID_ARGUMENT; ctx->fused_planes = (int)value; return OK; }
    if (!strcmp(name, "comm_timeout_ms")) { if (value < 1 || value > 3600000) return INVALID_ARGUMENT; ctx->comm_timeout_ms = value; return OK; }
    if (!strcmp(name, "time_steps")) { if (value < 0 || value > 1) return INVALID_ARGUMENT; ctx->time_steps = (int)value; return OK; }
    return INVALID_ARGUMENT;
}

int32_t synaptik_cuda_context_synchronize(void *context) {
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx) return INVALID_ARGUMENT;
    DeviceGuard guard(ctx->device);
    cudaError_t e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->comm_stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->copy_stream);
    return cuda_status(e, EXECUTION_FAILED);
}

int32_t synaptik_cuda_context_timer_start(void *context) {
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx) return INVALID_ARGUMENT;
    DeviceGuard guard(ctx->device);
    if (!ctx->timer_start && (cudaEventCreate(&ctx->timer_start) != cudaSuccess || cudaEventCreate(&ctx->timer_stop) != cudaSuccess)) return INTERNAL_ERROR;
    return cuda_status(cudaEventRecord(ctx->timer_start, ctx->stream), EXECUTION_FAILED);
}

int32_t synaptik_cuda_context_timer_stop(void *context, double *out_milliseconds) {
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx || !out_milliseconds || !ctx->timer_start) return INVALID_ARGUMENT;
    DeviceGuard guard(ctx->device);
    float ms = 0;
    cudaError_t e = cudaEventRecord(ctx->timer_stop, ctx->stream);
    if (e == cudaSuccess) e = cudaEventSynchronize(ctx->timer_stop);
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, ctx->timer_start, ctx->timer_stop);
    if (e != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
    *out_milliseconds = ms;
    return OK;
}

int32_t synaptik_cuda_buffer_create(void *context, uint64_t bytes, void **out_buffer) {
    if (!out_buffer) return INVALID_ARGUMENT;
    *out_buffer = nullptr;
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx) return INVALID_ARGUMENT;
    DeviceGuard guard(ctx->device);
    void *p = nullptr;
    if (cudaMalloc(&p, bytes ? bytes : 4) != cudaSuccess) { cudaGetLastError(); return ALLOCATION_FAILED; }
    Buffer *b = new Buffer();
    b->ctx = ctx; b->ptr = p; b->bytes = bytes;
    *out_buffer = b;
    return OK;
}

int32_t synaptik_cuda_buffer_release(void *buffer) {
    Buffer *b = as<Buffer>(buffer, TAG_BUFFER);
    if (!b) return INVALID_ARGUMENT;
    DeviceGuard guard(b->ctx->device);
    cudaStreamSynchronize(b->ctx->stream);
    cudaStreamSynchronize(b->ctx->copy_stream);
    if (b->filled) cudaEventDestroy(b->filled);
    if (b->released) cudaEventDestroy(b->released);
    cudaFree(b->ptr);
    b->tag = 0;
    delete b;
    return OK;
}

static int32_t transfer(void *buffer, uint64_t offset, void *host, uint64_t bytes, bool upload, bool async) {
    Buffer *b = as<Buffer>(buffer, TAG_BUFFER);
    if (!b || (!host && bytes)) return INVALID_ARGUMENT;
    if (offset > b->bytes || bytes > b->bytes - offset) return RANGE_OUT_OF_BOUNDS;
    if (!bytes) return OK;
    std::lock_guard<std::mutex> lock(b->ctx->mutex);
    DeviceGuard guard(b->ctx->device);
    uint8_t *dev = (uint8_t *)b->ptr + offset;
    if (b->fill_pending) { cudaStreamWaitEvent(b->ctx->stream, b->filled, 0); b->fill_pending = false; }
    cudaError_t e = upload ? cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, b->ctx->stream)
                           : cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, b->ctx->stream);
    if (e == cudaSuccess && !async) e = cudaStreamSynchronize(b->ctx->stream);
    // a later prefetch into this buffer has to wait for a copy that is still in flight
    if (e == cudaSuccess && async && b->released) { cudaEventRecord(b->released, b->ctx->stream); b->release_recorded = true; }
    if (e != cudaSuccess) { cudaGetLastError(); return COPY_FAILED; }
    return OK;
}

int32_t synaptik_cuda_buffer_upload(void *buffer, uint64_t offset, const void *source, uint64_t bytes) {
    return transfer(buffer, offset, const_cast<void *>(source), bytes, true, false);
}
int32_t synaptik_cuda_buffer_download(void *buffer, uint64_t offset, void *destination, uint64_t bytes) {
    return transfer(buffer, offset, destination, bytes, false, false);
}
int32_t synaptik_cuda_buffer_upload_async(void *buffer, uint64_t offset, const void *source, uint64_t bytes) {
    return transfer(buffer, offset, const_cast<void *>(source), bytes, true, true);
}
int32_t synaptik_cuda_buffer_download_async(void *buffer, uint64_t offset, void *destination, uint64_t bytes) {
    return transfer(buffer, offset, destination, bytes, false, true);
}

int32_t synaptik_cuda_buffer_prefetch(void *buffer, uint64_t offset, const void *source, uint64_t bytes) {
    Buffer *b = as<Buffer>(buffer, TAG_BUFFER);
    if (!b || (!source && bytes)) return INVALID_ARGUMENT;
    if (offset > b->bytes || bytes > b->bytes - offset) return RANGE_OUT_OF_BOUNDS;
    if (!bytes) return OK;
    Context *ctx = b->ctx;
    std::lock_guard<std::mutex> lock(ctx->mutex);
    DeviceGuard guard(ctx->device);
    if (!b->filled && (cudaEventCreateWithFlags(&b->filled, cudaEventDisableTiming) != cudaSuccess
                       || cudaEventCreateWithFlags(&b->released, cudaEventDisableTiming) != cudaSuccess)) { cudaGetLastError(); return INTERNAL_ERROR; }
    // The copy may not overtake the runs and copies already enqueued that read or write this buffer.
    // Runs record `released` only for buffers that have these events, so the first prefetch into a
    // buffer records it here, behind everything the compute stream holds so far.
    cudaError_t e = cudaSuccess;
    if (!b->release_recorded) { e = cudaEventRecord(b->released, ctx->stream); b->release_recorded = true; }
    if (e == cudaSuccess) e = cudaStreamWaitEvent(ctx->copy_stream, b->released, 0);
    if (e == cudaSuccess) e = cudaMemcpyAsync((uint8_t *)b->ptr + offset, source, bytes, cudaMemcpyHostToDevice, ctx->copy_stream);
    if (e == cudaSuccess) e = cudaEventRecord(b->filled, ctx->copy_stream);
    if (e != cudaSuccess) { cudaGetLastError(); return COPY_FAILED; }
    b->fill_pending = true;
    return OK;
}

int32_t synaptik_cuda_buffer_upload_canonical(void *buffer, uint64_t offset, const void *source, uint64_t bytes, uint32_t element_bytes) {
    if (element_bytes != 1 && element_bytes != 2 && element_bytes != 4 && element_bytes != 8) return INVALID_ARGUMENT;
    if (bytes % element_bytes) return INVALID_ARGUMENT;
    Buffer *b = as<Buffer>(buffer, TAG_BUFFER);
    if (!b || (!source && bytes)) return INVALID_ARGUMENT;
    if (offset > b->bytes || bytes > b->bytes - offset) return RANGE_OUT_OF_BOUNDS;
    std::vector<uint8_t> staged(bytes);
    bswap_copy(staged.data(), (const uint8_t *)source, bytes, element_bytes);
    return transfer(buffer, offset, staged.data(), bytes, true, false);
}

int32_t synaptik_cuda_buffer_download_canonical(void *buffer, uint64_t offset, void *destination, uint64_t bytes, uint32_t element_bytes) {
    if (element_bytes != 1 && element_bytes != 2 && element_bytes != 4 && element_bytes != 8) return INVALID_ARGUMENT;
    if (bytes % element_bytes) return INVALID_ARGUMENT;
    Buffer *b = as<Buffer>(buffer, TAG_BUFFER);
    if (!b || (!destination && bytes)) return INVALID_ARGUMENT;
    if (offset > b->bytes || bytes > b->bytes - offset) return RANGE_OUT_OF_BOUNDS;
    std::vector<uint8_t> staged(bytes);
    int32_t s = transfer(buffer, offset, staged.data(), bytes, false, false);
    if (s != OK) return s;
    bswap_copy((uint8_t *)destination, staged.data(), bytes, element_bytes);
    return OK;
}

int32_t synaptik_cuda_buffer_device_pointer(void *buffer, uint64_t *out_address, uint64_t *out_bytes) {
    Buffer *b = as<Buffer>(buffer, TAG_BUFFER);
    if (!b || !out_address) return INVALID_ARGUMENT;
    *out_address = (uint64_t)(uintptr_t)b->ptr;
    if (out_bytes) *out_bytes = b->bytes;
    return OK;
}

int32_t synaptik_cuda_host_alloc(uint64_t bytes, void **out_pointer) {
    if (!out_pointer) return INVALID_ARGUMENT;
    *out_pointer = nullptr;
    void *p = nullptr;
    cudaError_t e = cudaMallocHost(&p, bytes ? bytes : 4);
    if (e != cudaSuccess) { cudaGetLastError(); return cuda_status(e, ALLOCATION_FAILED); }
    *out_pointer = p;
    return OK;
}
int32_t synaptik_cuda_host_free(void *pointer) {
    if (!pointer) return INVALID_ARGUMENT;
    cudaError_t e = cudaFreeHost(pointer);
    if (e != cudaSuccess) { cudaGetLastError(); return INVALID_ARGUMENT; }
    return OK;
}

int32_t synaptik_cuda_executable_create(void *context, const uint8_t *program, uint32_t program_bytes, void **out_executable) {
    if (!out_executable) return INVALID_ARGUMENT;
    *out_executable = nullptr;
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx || !program) return INVALID_ARGUMENT;
    Executable *x = new Executable();
    x->ctx = ctx;
    int32_t s = build_program(program, program_bytes, ctx->gemm_engine, x->program, x->plan);
    if (s != OK) { delete x; return s; }
    DeviceGuard guard(ctx->device);
    s = prepare_executable(x);
    if (s != OK) { release_executable(x); return s; }
    *out_executable = x;
    return OK;
}

int32_t synaptik_cuda_executable_release(void *executable) {
    Executable *x = as<Executable>(executable, TAG_EXECUTABLE);
    if (!x) return INVALID_ARGUMENT;
    release_executable(x);
    return OK;
}

int32_t synaptik_cuda_executable_enqueue(void *executable, int32_t input_count, void *const *inputs, int32_t output_count, void *const *outputs) {
    Executable *x = as<Executable>(executable, TAG_EXECUTABLE);
    if (!x) return INVALID_ARGUMENT;
    Binding bind;
    int32_t s = bind_buffers(x, input_count, inputs, output_count, outputs, bind);
    if (s != OK) return s;
    std::lock_guard<std::mutex> lock(x->ctx->mutex);
    DeviceGuard guard(x->ctx->device);
    return enqueue_executable(x, bind);
}

int32_t synaptik_cuda_executable_finish(void *executable) {
    Executable *x = as<Executable>(executable, TAG_EXECUTABLE);
    if (!x) return INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(x->ctx->mutex);
    DeviceGuard guard(x->ctx->device);
    x->pending = false;
    return drain_errors(x->ctx);
}

int32_t synaptik_cuda_executable_run(void *executable, int32_t input_count, void *const *inputs, int32_t output_count, void *const *outputs) {
    int32_t s = synaptik_cuda_executable_enqueue(executable, input_count, inputs, output_count, outputs);
    if (s != OK) return s;
    return synaptik_cuda_executable_finish(executable);
}

int32_t synaptik_cuda_program_describe(const uint8_t *program, uint32_t program_bytes, char *text, uint64_t capacity, uint64_t *out_required) {
    if (!program) return INVALID_ARGUMENT;
    Program g; Plan plan;
    int32_t s = build_program(program, program_bytes, 0, g, plan);
    if (s != OK) return s;
    std::string d = describe_plan(g, plan);
    if (out_required) *out_required = d.size() + 1;
    if (!text || capacity < d.size() + 1) return INVALID_ARGUMENT;
    memcpy(text, d.c_str(), d.size() + 1);
    return OK;
}

int32_t synaptik_cuda_executable_describe(void *executable, char *text, uint64_t capacity, uint64_t *out_required) {
    Executable *x = as<Executable>(executable, TAG_EXECUTABLE);
    if (!x) return INVALID_ARGUMENT;
    std::string d = describe_plan(x->program, x->plan);
    if (out_required) *out_required = d.size() + 1;
    if (!text || capacity < d.size() + 1) return INVALID_ARGUMENT;
    memcpy(text, d.c_str(), d.size() + 1);
    return OK;
}

int32_t synaptik_cuda_executable_step_timings(void *executable, double *out_milliseconds, uint64_t capacity, uint64_t *out_count) {
    Executable *x = as<Executable>(executable, TAG_EXECUTABLE);
    if (!x || !out_count) return INVALID_ARGUMENT;
    size_t steps = x->plan.steps.size();
    *out_count = steps;
    if (!x->steps_timed || !x->timed) return INVALID_ARGUMENT;
    if (!out_milliseconds || capacity < steps) return INVALID_ARGUMENT;
    DeviceGuard guard(x->ctx->device);
    if (cudaEventSynchronize(x->stop) != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
    for (size_t i = 0; i < steps; i++) {
        float ms = 0;
        if (cudaEventElapsedTime(&ms, x->step_events[2 * i], x->step_events[2 * i + 1]) != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
        out_milliseconds[i] = ms;
    }
    return OK;
}

int32_t synaptik_cuda_executable_last_timing(void *executable, double *out_milliseconds) {
    Executable *x = as<Executable>(executable, TAG_EXECUTABLE);
    if (!x || !out_milliseconds || !x->timed) return INVALID_ARGUMENT;
    DeviceGuard guard(x->ctx->device);
    float ms = 0;
    if (cudaEventSynchronize(x->stop) != cudaSuccess || cudaEventElapsedTime(&ms, x->start, x->stop) != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
    *out_milliseconds = ms;
    return OK;
}

int32_t synaptik_cuda_executable_launch_count(void *executable, uint64_t *out_launches) {
    Executable *x = as<Executable>(executable, TAG_EXECUTABLE);
    if (!x || !out_launches) return INVALID_ARGUMENT;
    *out_launches = x->launches;
    return OK;
}

// ---- optimizer -----------------------------------------------------------------------------------
int32_t synaptik_cuda_optimizer_create(void *context, int32_t kind, const double *hyper, int32_t hyper_count, int32_t parameter_count,
                                       void *const *parameters, const uint64_t *element_counts, void **out_optimizer) {
    if (!out_optimizer) return INVALID_ARGUMENT;
    *out_optimizer = nullptr;
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx || kind < 0 || kind > 2 || !hyper || hyper_count != 5 || parameter_count < 1 || !parameters || !element_counts) return INVALID_ARGUMENT;
    for (int i = 0; i < 5; i++) if (!std::isfinite(hyper[i])) return INVALID_ARGUMENT;
    if (kind == 0) { if (!(hyper[0] > 0) || hyper[1] < 0 || hyper[3] < 0) return INVALID_ARGUMENT; }
    else if (!(hyper[0] > 0) || hyper[1] < 0 || hyper[1] >= 1 || hyper[2] < 0 || hyper[2] >= 1 || !(hyper[3] > 0) || hyper[4] < 0) return INVALID_ARGUMENT;
    Optimizer *o = new Optimizer();
    o->ctx = ctx; o->kind = kind;
    memcpy(o->hyper, hyper, sizeof o->hyper);
    DeviceGuard guard(ctx->device);
    bool need_m = kind != 0 || hyper[1] != 0.0, need_v = kind != 0;
    int32_t status = OK;
    std::lock_guard<std::mutex> lock(ctx->mutex);
    auto zeroed = [&](uint64_t bytes, float **out) {
        if (cudaMalloc(out, bytes) != cudaSuccess || cudaMemsetAsync(*out, 0, bytes, ctx->stream) != cudaSuccess) status = ALLOCATION_FAILED;
    };
    for (int i = 0; i < parameter_count && status == OK; i++) {
        Buffer *b = as<Buffer>(parameters[i], TAG_BUFFER);
        if (!b) { status = INVALID_ARGUMENT; break; }
        if (b->ctx != ctx || b->bytes < element_counts[i] * 4) { status = INCOMPATIBLE_RESOURCE; break; }
        o->params.push_back(b); o->counts.push_back(element_counts[i]);
        float *m = nullptr, *v = nullptr, *p2 = nullptr, *m2 = nullptr, *v2 = nullptr;
        uint64_t bytes = element_counts[i] ? element_counts[i] * 4 : 4;
        if (need_m) { zeroed(bytes, &m); if (status == OK) zeroed(bytes, &m2); }
        if (status == OK && need_v) { zeroed(bytes, &v); if (status == OK) zeroed(bytes, &v2); }
        // the second parameter array has the buffer's full size and starts as a copy of it, so whatever the
        // buffer holds past the parameter's elements is in both
        if (status == OK && (cudaMalloc(&p2, b->bytes ? b->bytes : 4) != cudaSuccess
                             || (b->bytes && cudaMemcpyAsync(p2, b->ptr, b->bytes, cudaMemcpyDeviceToDevice, ctx->stream) != cudaSuccess))) status = ALLOCATION_FAILED;
        o->m.push_back(m); o->v.push_back(v); o->p_alt.push_back(p2); o->m_alt.push_back(m2); o->v_alt.push_back(v2);
    }
    if (status == OK && (cudaMalloc(&o->failed_dev, sizeof(int)) != cudaSuccess || cudaMemsetAsync(o->failed_dev, 0x7f, sizeof(int), ctx->stream) != cudaSuccess)) status = ALLOCATION_FAILED;
    if (status == OK && cudaStreamSynchronize(ctx->stream) != cudaSuccess) status = EXECUTION_FAILED;
    if (status != OK) {
        cudaGetLastError();
        for (auto *set : {&o->m, &o->v, &o->p_alt, &o->m_alt, &o->v_alt}) for (float *q : *set) cudaFree(q);
        cudaFree(o->failed_dev);
        delete o;
        return status;
    }
    ctx->optimizers.push_back(o);
    *out_optimizer = o;
    return OK;
}

int32_t synaptik_cuda_optimizer_release(void *optimizer) {
    Optimizer *o = as<Optimizer>(optimizer, TAG_OPTIMIZER);
    if (!o) return INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(o->ctx->mutex);
    DeviceGuard guard(o->ctx->device);
    // steps still in flight are settled first, so the parameter buffers are left holding a committed state
    if (!o->journal.empty()) drain_errors(o->ctx);
    else cudaStreamSynchronize(o->ctx->stream);
    auto &list = o->ctx->optimizers;
    list.erase(std::remove(list.begin(), list.end(), o), list.end());
    for (auto *set : {&o->m, &o->v, &o->p_alt, &o->m_alt, &o->v_alt, &o->acc}) for (float *q : *set) cudaFree(q);
    cudaFree(o->failed_dev);
    o->tag = 0;
    delete o;
    return OK;
}

static int32_t optimizer_enqueue(void *optimizer, int32_t mode, int32_t gradient_count, void *const *gradients) {
    Optimizer *o = as<Optimizer>(optimizer, TAG_OPTIMIZER);
    if (!o || gradient_count != (int32_t)o->params.size() || !gradients || mode < 0 || mode > 2) return INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(o->ctx->mutex);
    DeviceGuard guard(o->ctx->device);
    if (mode != 0 && o->acc.empty()) {
        // pending sums start at zero (TrainingParameter.java:103-109)
        for (size_t i = 0; i < o->params.size(); i++) {
            void *p = nullptr;
            uint64_t bytes = o->counts[i] ? o->counts[i] * 4 : 4;
            if (cudaMalloc(&p, bytes) != cudaSuccess) { cudaGetLastError(); for (float *q : o->acc) cudaFree(q); o->acc.clear(); return ALLOCATION_FAILED; }
            cudaMemsetAsync(p, 0, bytes, o->ctx->stream);
            o->acc.push_back((float *)p);
        }
    }
    if (o->journal.size() >= 65536) {        // a caller that never finishes: settle what is in flight
        int32_t settled = drain_errors(o->ctx);
        if (settled != OK) return settled;
    }
    std::vector<kern::TensorSlot> slots(o->params.size());
    for (size_t i = 0; i < slots.size(); i++) {
        Buffer *g = as<Buffer>(gradients[i], TAG_BUFFER);
        if (!g) return INVALID_ARGUMENT;
        if (g->ctx != o->ctx || g->bytes < o->counts[i] * 4 || g == o->params[i]) return INCOMPATIBLE_RESOURCE;
        slots[i] = {(const float *)o->params[i]->ptr, (const float *)g->ptr, o->m[i], o->v[i], (int64_t)o->counts[i],
                    o->acc.empty() ? nullptr : o->acc[i], o->p_alt[i], o->m_alt[i], o->v_alt[i]};
    }
    cudaError_t e;
    cudaStream_t stream = o->ctx->stream;
    const int sequence = (int)o->journal.size();
    const Optimizer::Entry before{mode != 1, o->steps, o->accumulated_runs, o->acc_dirty};
    if (mode == 1) {
        e = kern::accumulate_gradients(stream, slots.data(), (int)slots.size(), sequence, o->failed_dev, o->ctx->error_dev);
        if (e != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
        o->journal.push_back(before);
        o->accumulated_runs++;
        o->acc_dirty = true;
        o->pending = true;
        return OK;
    }
    if (o->kind == 0) {
        kern::SgdArgs a;
        a.lr = (float)o->hyper[0]; a.momentum = (float)o->hyper[1]; a.dampening = (float)o->hyper[2]; a.weight_decay = (float)o->hyper[3];
        a.nesterov = o->hyper[4] != 0.0; a.first_step = o->steps == 0; a.has_buffer = o->hyper[1] != 0.0;
        a.zero_buffer = o->hyper[1] != 0.0 && a.momentum == 0.0f;
        a.gradient_mode = mode; a.sequence = sequence; a.failed_sequence = o->failed_dev;
        e = kern::sgd_step(stream, slots.data(), (int)slots.size(), a, o->ctx->error_dev);
    } else {
        // coefficients narrowed to binary32 first (AdaptiveCoefficients.java:33-58); corrections
        // 1f - (float)Math.pow(beta, step) evaluated in binary64 on the narrowed beta
        kern::AdamArgs a;
        a.lr = (float)o->hyper[0]; a.b1 = (float)o->hyper[1]; a.b2 = (float)o->hyper[2]; a.eps = (float)o->hyper[3]; a.decay = (float)o->hyper[4];
        double step = (double)(o->steps + 1);
        a.correction1 = 1.0f - (float)std::pow((double)a.b1, step);
        a.correction2 = 1.0f - (float)std::pow((double)a.b2, step);
        if (!(a.correction1 > 0.0f) || !(a.correction2 > 0.0f)) return EXECUTION_FAILED;
        a.decoupled = o->kind == 2;
        a.decay_factor = 1.0f;
        if (a.decoupled) { float scale = a.lr * a.decay; a.decay_factor = 1.0f - scale; }
        a.gradient_mode = mode; a.sequence = sequence; a.failed_sequence = o->failed_dev;
        e = kern::adam_step(stream, slots.data(), (int)slots.size(), a, o->ctx->error_dev);
    }
    // the pending sum is consumed (ACCUMULATE_AND_STEP) or dropped (RESET_AND_STEP after accumulating
    // runs) only once the step has gone through: a second launch, which the error word turns into a no-op
    if (e == cudaSuccess && o->acc_dirty && !o->acc.empty()) e = kern::clear_pending(stream, slots.data(), (int)slots.size(), o->ctx->error_dev);
    if (e != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
    // The candidates become current at once, so that runs enqueued behind this step read them; the
    // exchange and the counters are taken back by the next drain if the step did not take place.
    o->journal.push_back(before);
    exchange_sets(o);
    o->steps++;
    o->accumulated_runs = 0;
    o->acc_dirty = false;
    o->pending = true;
    return OK;
}

int32_t synaptik_cuda_optimizer_step_enqueue(void *optimizer, int32_t gradient_count, void *const *gradients) {
    return optimizer_enqueue(optimizer, 0, gradient_count, gradients);
}

int32_t synaptik_cuda_optimizer_run_enqueue(void *optimizer, int32_t gradient_mode, int32_t gradient_count, void *const *gradients) {
    return optimizer_enqueue(optimizer, gradient_mode, gradient_count, gradients);
}

int32_t synaptik_cuda_optimizer_run(void *optimizer, int32_t gradient_mode, int32_t gradient_count, void *const *gradients) {
    int32_t s = optimizer_enqueue(optimizer, gradient_mode, gradient_count, gradients);
    if (s != OK) return s;
    return synaptik_cuda_optimizer_finish(optimizer);
}

int32_t synaptik_cuda_optimizer_zero_grad(void *optimizer) {
    Optimizer *o = as<Optimizer>(optimizer, TAG_OPTIMIZER);
    if (!o) return INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(o->ctx->mutex);
    DeviceGuard guard(o->ctx->device);
    for (size_t i = 0; i < o->acc.size(); i++)
        if (cudaMemsetAsync(o->acc[i], 0, o->counts[i] * 4, o->ctx->stream) != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
    o->accumulated_runs = 0;
    o->acc_dirty = false;
    return OK;
}

int32_t synaptik_cuda_optimizer_accumulated_runs(void *optimizer, uint64_t *out_runs) {
    Optimizer *o = as<Optimizer>(optimizer, TAG_OPTIMIZER);
    if (!o || !out_runs) return INVALID_ARGUMENT;
    *out_runs = o->accumulated_runs;
    return OK;
}

int32_t synaptik_cuda_optimizer_finish(void *optimizer) {
    Optimizer *o = as<Optimizer>(optimizer, TAG_OPTIMIZER);
    if (!o) return INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(o->ctx->mutex);
    DeviceGuard guard(o->ctx->device);
    o->pending = false;
    return drain_errors(o->ctx);
}

int32_t synaptik_cuda_optimizer_step(void *optimizer, int32_t gradient_count, void *const *gradients) {
    int32_t s = synaptik_cuda_optimizer_step_enqueue(optimizer, gradient_count, gradients);
    if (s != OK) return s;
    return synaptik_cuda_optimizer_finish(optimizer);
}

int32_t synaptik_cuda_optimizer_steps(void *optimizer, uint64_t *out_steps) {
    Optimizer *o = as<Optimizer>(optimizer, TAG_OPTIMIZER);
    if (!o || !out_steps) return INVALID_ARGUMENT;
    *out_steps = o->steps;
    return OK;
}

static int32_t optimizer_state(void *optimizer, int32_t index, int32_t slot, void *host, uint64_t bytes, bool upload, bool canonical) {
    Optimizer *o = as<Optimizer>(optimizer, TAG_OPTIMIZER);
    if (!o || index < 0 || index >= (int32_t)o->params.size() || slot < 0 || slot > 2 || !host) return INVALID_ARGUMENT;
    if (bytes != o->counts[index] * 4) return RANGE_OUT_OF_BOUNDS;
    std::lock_guard<std::mutex> lock(o->ctx->mutex);
    DeviceGuard guard(o->ctx->device);
    if (!o->journal.empty()) {              // steps still in flight: settle them first, so the state moved is a committed one
        int32_t settled = drain_errors(o->ctx);
        if (settled != OK) return settled;
    }
    if (slot == 2 && o->acc.empty()) {
        if (!upload) {                      // no run has accumulated yet: the pending sum is all zeros
            memset(host, 0, bytes);
            return OK;
        }
        for (size_t i = 0; i < o->params.size(); i++) {
            void *p = nullptr;
            uint64_t size = o->counts[i] ? o->counts[i] * 4 : 4;
            if (cudaMalloc(&p, size) != cudaSuccess) { cudaGetLastError(); for (float *q : o->acc) cudaFree(q); o->acc.clear(); return ALLOCATION_FAILED; }
            cudaMemsetAsync(p, 0, size, o->ctx->stream);
            o->acc.push_back((float *)p);
        }
    }
    float *dev = slot == 0 ? o->m[index] : slot == 1 ? o->v[index] : o->acc[index];
    if (!dev) return INVALID_ARGUMENT;
    std::vector<uint8_t> staged;
    void *side = host;
    if (canonical) {                        // big-endian FLOAT32 elements, TrainingParameter.java:894-941
        staged.resize(bytes);
        if (upload) bswap_copy(staged.data(), (const uint8_t *)host, bytes, 4);
        side = staged.data();
    }
    cudaError_t e = upload ? cudaMemcpyAsync(dev, side, bytes, cudaMemcpyHostToDevice, o->ctx->stream)
                           : cudaMemcpyAsync(side, dev, bytes, cudaMemcpyDeviceToHost, o->ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(o->ctx->stream);
    if (e != cudaSuccess) { cudaGetLastError(); return COPY_FAILED; }
    if (canonical && !upload) bswap_copy((uint8_t *)host, staged.data(), bytes, 4);
    if (upload && slot == 2) o->acc_dirty = true;
    return OK;
}
int32_t synaptik_cuda_optimizer_download_state(void *optimizer, int32_t parameter_index, int32_t slot, void *destination, uint64_t bytes) {
    return optimizer_state(optimizer, parameter_index, slot, destination, bytes, false, false);
}
int32_t synaptik_cuda_optimizer_upload_state(void *optimizer, int32_t parameter_index, int32_t slot, const void *source, uint64_t bytes, uint64_t completed_steps) {
    int32_t s = optimizer_state(optimizer, parameter_index, slot, const_cast<void *>(source), bytes, true, false);
    if (s == OK) as<Optimizer>(optimizer, TAG_OPTIMIZER)->steps = completed_steps;
    return s;
}
int32_t synaptik_cuda_optimizer_download_state_canonical(void *optimizer, int32_t parameter_index, int32_t slot, void *destination, uint64_t bytes) {
    return optimizer_state(optimizer, parameter_index, slot, destination, bytes, false, true);
}
int32_t synaptik_cuda_optimizer_upload_state_canonical(void *optimizer, int32_t parameter_index, int32_t slot, const void *source, uint64_t bytes) {
    return optimizer_state(optimizer, parameter_index, slot, const_cast<void *>(source), bytes, true, true);
}
int32_t synaptik_cuda_optimizer_set_progress(void *optimizer, uint64_t completed_steps, uint64_t accumulated_runs) {
    Optimizer *o = as<Optimizer>(optimizer, TAG_OPTIMIZER);
    if (!o) return INVALID_ARGUMENT;
    o->steps = completed_steps;
    o->accumulated_runs = accumulated_runs;
    return OK;
}

// ---- communicator --------------------------------------------------------------------------------
int32_t synaptik_cuda_comm_unique_id(uint8_t *out_id128) {
    if (!out_id128) return INVALID_ARGUMENT;
    if (!nccl().ok) return COMM_FAILED;
    NcclApi::UniqueId id;
    if (nccl().GetUniqueId(&id) != 0) return COMM_FAILED;
    memcpy(out_id128, id.internal, 128);
    return OK;
}

int32_t synaptik_cuda_comm_create(void *context, int32_t world_size, int32_t rank, const uint8_t *unique_id128, void **out_comm) {
    if (!out_comm) return INVALID_ARGUMENT;
    *out_comm = nullptr;
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx || world_size < 1 || rank < 0 || rank >= world_size || !unique_id128) return INVALID_ARGUMENT;
    if (!nccl().ok) return COMM_FAILED;
    DeviceGuard guard(ctx->device);
    NcclApi::UniqueId id;
    memcpy(id.internal, unique_id128, 128);
    void *comm = nullptr;
    if (nccl().CommInitRank(&comm, world_size, id, rank) != 0 || !comm) return COMM_FAILED;
    Comm *c = new Comm();
    c->ctx = ctx; c->comm = comm; c->world = world_size; c->rank = rank;
    {
        std::lock_guard<std::mutex> lock(ctx->mutex);
        ctx->comms.push_back(c);
    }
    *out_comm = c;
    return OK;
}

int32_t synaptik_cuda_comm_release(void *comm) {
    Comm *c = as<Comm>(comm, TAG_COMM);
    if (!c) return INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(c->ctx->mutex);
    DeviceGuard guard(c->ctx->device);
    cudaStreamSynchronize(c->ctx->comm_stream);
    if (c->comm) nccl().CommDestroy(c->comm);       // an aborted communicator is already gone
    auto &list = c->ctx->comms;
    list.erase(std::remove(list.begin(), list.end(), c), list.end());
    c->tag = 0;
    delete c;
    return OK;
}

int32_t synaptik_cuda_comm_allreduce_sum_f32(void *comm, void *buffer, uint64_t offset, uint64_t element_count) {
    Comm *c = as<Comm>(comm, TAG_COMM);
    Buffer *b = as<Buffer>(buffer, TAG_BUFFER);
    if (!c || !b) return INVALID_ARGUMENT;
    if (b->ctx != c->ctx) return INCOMPATIBLE_RESOURCE;
    if (offset % 4 || offset > b->bytes || element_count * 4 > b->bytes - offset) return RANGE_OUT_OF_BOUNDS;
    std::lock_guard<std::mutex> lock(c->ctx->mutex);
    DeviceGuard guard(c->ctx->device);
    if (c->dead) return COMM_FAILED;
    // ordered after the compute stream's earlier work, executed on the communication stream, and the
    // compute stream continues behind it
    cudaEvent_t ev;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return INTERNAL_ERROR;
    cudaEventRecord(ev, c->ctx->stream);
    cudaStreamWaitEvent(c->ctx->comm_stream, ev, 0);
    float *p = (float *)((uint8_t *)b->ptr + offset);
    int rc = nccl().AllReduce(p, p, element_count, 7, 0, c->comm, c->ctx->comm_stream);
    cudaEventRecord(ev, c->ctx->comm_stream);
    cudaStreamWaitEvent(c->ctx->stream, ev, 0);
    // the host waits with the context's deadline; whatever else was in flight on the context is settled too
    int32_t status = drain_errors(c->ctx);
    cudaEventDestroy(ev);
    if (rc != 0) return COMM_FAILED;
    return status;
}

int32_t synaptik_cuda_executable_attach_comm(void *executable, void *comm, int32_t output_count, const int32_t *output_indices) {
    Executable *x = as<Executable>(executable, TAG_EXECUTABLE);
    if (!x) return INVALID_ARGUMENT;
    if (!comm) { x->comm = nullptr; x->sync_publication.assign(x->program.publications.size(), 0); return OK; }
    Comm *c = as<Comm>(comm, TAG_COMM);
    if (!c || output_count < 0 || (output_count && !output_indices)) return INVALID_ARGUMENT;
    if (c->ctx != x->ctx) return INCOMPATIBLE_RESOURCE;
    std::vector<char> flags(x->program.publications.size(), 0);
    for (int i = 0; i < output_count; i++) {
        int j = output_indices[i];
        if (j < 0 || j >= (int)flags.size()) return INVALID_ARGUMENT;
        if (x->program.values[x->program.publications[j]].dtype != DType::F32) return INCOMPATIBLE_RESOURCE;
        flags[j] = 1;
    }
    // The reduction runs in place on the communication stream as soon as the publication is final, while
    // the compute stream goes on: a publication that a later step of the plan still reads would be read
    // half reduced.
    for (size_t ready = 0; ready < x->plan.steps.size(); ready++)
        for (int j : x->plan.steps[ready].ready_publications) {
            if (!flags[j]) continue;
            for (size_t later = ready + 1; later < x->plan.steps.size(); later++) {
                const Step &st = x->plan.steps[later];
                for (int value : {st.a, st.b, st.c, st.bias, st.mask}) {
                    if (value < 0) continue;
                    const View &v = x->plan.views[value];
                    if (v.slot == SlotKind::PUBLICATION && v.index == j) return INCOMPATIBLE_RESOURCE;
                }
            }
        }
    // An all-reduce that overlaps the backward pass holds some SMs.  A product of one wave or less cannot give
    // way to it (its tiles then take two waves: measured 0.45 ms instead of 0.24 for a 784 x 4096 x 8192 weight
    // gradient with 24 SMs held), so such epilogue-free products are planned again in slices (0.36 ms).
    if (x->ctx->gemm_slices == 1) {
        std::lock_guard<std::mutex> lock(x->ctx->mutex);
        DeviceGuard guard(x->ctx->device);
        bool synced = false;
        for (size_t i = 0; i < x->exec.size(); i++) {
            StepExec &se = x->exec[i];
            if (!se.tc || !se.tc_plain || se.emit_planes >= 0 || !kern::tc_gemm_single_wave(se.tc)) continue;    // (a sliced product has no epilogue to write planes from)
            int status = OK;
            kern::TensorCoreGemm *again = kern::tc_gemm_prepare(se.tc_p, se.tc_q, se.tc_m, se.tc_n, x->plan.steps[i].k, x->ctx->sm_count, se.tc_mode | 4 | 8, &status);
            if (!again) continue;
            if (kern::tc_gemm_launches(again) < 2) { kern::tc_gemm_release(again); continue; }
            const int64_t need = kern::tc_gemm_workspace_floats(again);
            if (!synced) { cudaStreamSynchronize(x->ctx->stream); synced = true; }       // no run of the old plan is in flight
            if (need > x->gemm_workspace_floats) {
                void *p = nullptr;
                if (cudaMalloc(&p, (uint64_t)need * 4) != cudaSuccess) { cudaGetLastError(); kern::tc_gemm_release(again); continue; }
                x->owned.push_back(p);
                x->gemm_workspace = (float *)p; x->gemm_workspace_floats = need;
            }
            kern::tc_gemm_release(se.tc);
            se.tc = again;
        }
    }
    x->comm = c;
    x->sync_publication = flags;
    return OK;
}

// Runs the give-up path of the device-side waits on purpose (see kern::wait_probe): the status is TIMEOUT
// and the context stays usable.
int32_t synaptik_cuda_context_wait_probe(void *context, uint64_t limit_microseconds) {
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx || limit_microseconds < 1 || limit_microseconds > 2000000) return INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(ctx->mutex);
    DeviceGuard guard(ctx->device);
    if (kern::wait_probe(ctx->stream, limit_microseconds * 1000ull, ctx->error_dev) != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
    return drain_errors(ctx);
}

// Co-tenant on the communication stream (see kern::occupy): asynchronous, ends by itself.
int32_t synaptik_cuda_context_occupy(void *context, int32_t blocks, uint64_t hold_microseconds) {
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    if (!ctx || blocks < 0 || blocks > ctx->sm_count || hold_microseconds > 100000) return INVALID_ARGUMENT;
    std::lock_guard<std::mutex> lock(ctx->mutex);
    DeviceGuard guard(ctx->device);
    if (kern::occupy(ctx->comm_stream, blocks, hold_microseconds * 1000ull) != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
    return OK;
}

// Column sums whose scratch lives in a static device array: no allocation of any kind on this path
// (no device or pinned memory, no containers).
int32_t synaptik_cuda_column_sums_no_alloc(void *context, void *input, uint64_t rows, uint64_t cols, void *output) {
    Context *ctx = as<Context>(context, TAG_CONTEXT);
    Buffer *in = as<Buffer>(input, TAG_BUFFER), *out = as<Buffer>(output, TAG_BUFFER);
    if (!ctx || !in || !out) return INVALID_ARGUMENT;
    if (in->ctx != ctx || out->ctx != ctx || in == out) return INCOMPATIBLE_RESOURCE;
    if (rows > (1ull << 40) || cols > (1ull << 30)) return UNSUPPORTED_SHAPE;
    if (rows * cols * 4 > in->bytes || cols * 4 > out->bytes) return RANGE_OUT_OF_BOUNDS;
    if (kern::colsum_partial_count((int64_t)rows, (int64_t)cols) > kern::kStaticColsumPartials) return UNSUPPORTED_SHAPE;
    std::lock_guard<std::mutex> lock(ctx->mutex);
    DeviceGuard guard(ctx->device);
    cudaError_t e = kern::colsum_static(ctx->stream, ctx->device, (const float *)in->ptr, (int64_t)rows, (int64_t)cols, (float *)out->ptr);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) { cudaGetLastError(); return EXECUTION_FAILED; }
    return OK;
}

}  // extern "C"
