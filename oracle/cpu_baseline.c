/*
 * Timed CPU baseline for the MLP path, shaped like the reference's CPU backend with its OpenBLAS
 * route enabled.  TEST / BENCHMARK INFRASTRUCTURE ONLY: never linked into the product library.
 *
 * What follows the reference:
 *  - GEMMs go to cblas_sgemm(RowMajor, NoTrans, NoTrans, m, n, k, 1, A, k, B, n, 0, C, n), the
 *    only call shape the reference issues (modules/backend/openblas-provider/.../
 *    OpenBlasGemmInvocation.java:41-68); a transposed operand is first copied to a dense
 *    row-major workspace, as the COPY_LEFT / COPY_RIGHT route plans do
 *    (modules/backend/cpu/.../route/nativeblas/openblas/CpuOpenBlasRoutePlan.java).
 *  - The library is looked up by the reference's own names (CpuOpenBlasDiscovery.java:125-152:
 *    "libopenblas.so.0", "libopenblas.so"), then by an explicit path given by the caller.
 *    Without any OpenBLAS the GEMM falls back to a threaded row loop and says so.
 *  - Bias add, ReLU, ReLU backward, bias gradient, softmax cross-entropy, and Adam are the scalar
 *    loops of synaptik_oracle.c (same citations), split over POSIX threads by index range when
 *    more than one thread is requested (the reference default is one thread,
 *    CpuBackendComposition.java:186,210).
 */
#define _GNU_SOURCE
#include <dlfcn.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>
#include <pthread.h>

#define SYN_EXPORT __attribute__((visibility("default")))

typedef void (*sgemm_fn)(int order, int transa, int transb, int m, int n, int k, float alpha,
        const float *a, int lda, const float *b, int ldb, float beta, float *c, int ldc);
typedef void (*set_threads_fn)(int);

static sgemm_fn g_sgemm = NULL;
static set_threads_fn g_set_threads = NULL;
static char g_blas_name[512] = "none (threaded row loop)";

/* Returns 1 when an OpenBLAS with unprefixed CBLAS symbols was bound. */
SYN_EXPORT int syn_baseline_bind_openblas(const char *explicit_path) {
    const char *names[] = {"libopenblas.so.0", "libopenblas.so", explicit_path};
    for (int i = 0; i < 3 && !g_sgemm; i++) {
        if (!names[i] || !names[i][0]) continue;
        void *h = dlopen(names[i], RTLD_NOW | RTLD_LOCAL);
        if (!h) continue;
        sgemm_fn f = (sgemm_fn)dlsym(h, "cblas_sgemm");
        if (!f) { dlclose(h); continue; }
        g_sgemm = f;
        g_set_threads = (set_threads_fn)dlsym(h, "openblas_set_num_threads");
        strncpy(g_blas_name, names[i], sizeof g_blas_name - 1);
    }
    return g_sgemm != NULL;
}

SYN_EXPORT const char *syn_baseline_blas_name(void) { return g_blas_name; }

static int g_threads = 1;
SYN_EXPORT void syn_baseline_set_threads(int threads) {
    g_threads = threads < 1 ? 1 : threads;
    if (g_set_threads) g_set_threads(g_threads);
}

/* Minimal fork-join over an index range: body(ctx, begin, end) on g_threads POSIX threads. */
typedef void (*range_fn)(void *ctx, int64_t begin, int64_t end);
typedef struct { range_fn fn; void *ctx; int64_t begin, end; } range_task;
static void *range_trampoline(void *arg) { range_task *t = (range_task *)arg; t->fn(t->ctx, t->begin, t->end); return NULL; }
static void parallel_range(int64_t count, range_fn fn, void *ctx) {
    int threads = g_threads;
    if (threads > count) threads = count > 0 ? (int)count : 1;
    if (threads <= 1) { fn(ctx, 0, count); return; }
    pthread_t *ids = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
    range_task *tasks = (range_task *)malloc(sizeof(range_task) * (size_t)threads);
    for (int t = 0; t < threads; t++) {
        tasks[t].fn = fn; tasks[t].ctx = ctx;
        tasks[t].begin = count * t / threads; tasks[t].end = count * (t + 1) / threads;
        if (t + 1 < threads) pthread_create(&ids[t], NULL, range_trampoline, &tasks[t]);
    }
    range_trampoline(&tasks[threads - 1]);
    for (int t = 0; t + 1 < threads; t++) pthread_join(ids[t], NULL);
    free(ids); free(tasks);
}

typedef struct { int m, n, k; const float *a, *b; float *c; } gemm_ctx;
static void gemm_rows(void *p, int64_t begin, int64_t end) {
    gemm_ctx *g = (gemm_ctx *)p;
    for (int64_t i = begin; i < end; i++) {
        float *ci = g->c + (size_t)i * g->n;
        for (int j = 0; j < g->n; j++) ci[j] = 0.0f;
        for (int q = 0; q < g->k; q++) {
            float av = g->a[(size_t)i * g->k + q]; const float *bp = g->b + (size_t)q * g->n;
            for (int j = 0; j < g->n; j++) ci[j] += av * bp[j];
        }
    }
}
static void gemm_nn(int m, int n, int k, const float *a, const float *b, float *c) {
    if (g_sgemm) { g_sgemm(101, 111, 111, m, n, k, 1.0f, a, k, b, n, 0.0f, c, n); return; }
    gemm_ctx g = {m, n, k, a, b, c};
    parallel_range(m, gemm_rows, &g);
}

typedef struct { int rows, cols; const float *src; float *dst; } transpose_ctx;
static void transpose_blocks(void *p, int64_t begin, int64_t end) {
    transpose_ctx *t = (transpose_ctx *)p;
    for (int64_t ib = begin; ib < end; ib++) {
        int i0 = (int)ib * 32;
        for (int j0 = 0; j0 < t->cols; j0 += 32)
            for (int i = i0; i < t->rows && i < i0 + 32; i++)
                for (int j = j0; j < t->cols && j < j0 + 32; j++)
                    t->dst[(size_t)j * t->rows + i] = t->src[(size_t)i * t->cols + j];
    }
}
static void transpose_copy(int rows, int cols, const float *src, float *dst) {
    transpose_ctx t = {rows, cols, src, dst};
    parallel_range((rows + 31) / 32, transpose_blocks, &t);
}

static double now_seconds(void) {
    struct timespec ts; clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

typedef struct { int n, relu; float *z; const float *b; } bias_ctx;
static void bias_rows(void *p, int64_t begin, int64_t end) {
    bias_ctx *c = (bias_ctx *)p;
    for (int64_t i = begin; i < end; i++) for (int j = 0; j < c->n; j++) {
        float v = c->z[(size_t)i * c->n + j] + c->b[j];
        if (c->relu) v = v != v ? v : (v > 0.0f ? v : 0.0f);
        c->z[(size_t)i * c->n + j] = v;
    }
}

typedef struct { int classes; const float *logits; const int32_t *labels; float *dz; float scale; double *row_loss; } ce_ctx;
static void ce_rows(void *p, int64_t begin, int64_t end) {
    ce_ctx *c = (ce_ctx *)p; int classes = c->classes;
    for (int64_t i = begin; i < end; i++) {
        const float *v = c->logits + (size_t)i * classes; float *d = c->dz + (size_t)i * classes;
        float maximum = -INFINITY;
        for (int k = 0; k < classes; k++) if (v[k] > maximum) maximum = v[k];
        float sum = 0.0f;
        for (int k = 0; k < classes; k++) { float s = v[k] - maximum; sum += (float)exp((double)s); }
        float lse = maximum + (float)log((double)sum);
        c->row_loss[i] = (double)(lse - v[c->labels[i]]);
        for (int k = 0; k < classes; k++) {
            float s = v[k] - maximum;
            float pr = (float)exp((double)s) / sum;
            d[k] = (pr - (k == c->labels[i] ? 1.0f : 0.0f)) * c->scale;
        }
    }
}

typedef struct { int rows, n; const float *dz; float *db; } colsum_ctx;
static void colsum_cols(void *p, int64_t begin, int64_t end) {
    colsum_ctx *c = (colsum_ctx *)p;
    for (int64_t j = begin; j < end; j++) {
        double s = 0.0;
        for (int i = 0; i < c->rows; i++) s += (double)c->dz[(size_t)i * c->n + j];
        c->db[j] = (float)s;
    }
}

typedef struct { const float *y; float *da; } mask_ctx;
static void mask_range(void *p, int64_t begin, int64_t end) {
    mask_ctx *c = (mask_ctx *)p;
    for (int64_t i = begin; i < end; i++) c->da[i] = c->y[i] > 0.0f ? c->da[i] : 0.0f;
}

typedef struct { float *p, *mm, *vv; const float *g; float lr, b1, b2, eps, c1, c2; } adam_ctx;
static void adam_range(void *q, int64_t begin, int64_t end) {
    adam_ctx *c = (adam_ctx *)q;
    for (int64_t i = begin; i < end; i++) {
        float gi = c->g[i];
        float m = c->b1 * c->mm[i] + (1.0f - c->b1) * gi;
        float v = c->b2 * c->vv[i] + (1.0f - c->b2) * (gi * gi);
        float mh = m / c->c1, vh = v / c->c2;
        float den = (float)sqrt((double)vh) + c->eps;
        c->p[i] = c->p[i] - (c->lr * mh) / den;
        c->mm[i] = m; c->vv[i] = v;
    }
}

/*
 * One MLP step on `rows` samples: forward through `layers` Linear layers (ReLU between them),
 * and, when `train` is non-zero, mean softmax cross-entropy, the full backward pass and one Adam
 * update (step number `adam_step`).  dims has layers+1 entries.  weights[l] is [dims[l+1],
 * dims[l]] row-major (the Linear storage, extensions/nn/.../layers/Linear.java:132-139),
 * biases[l] is [dims[l+1]].  m1/m2 hold the Adam moments as [w0,b0,w1,b1,...].  The gradient
 * scale is 1/count_total (global batch).  Returns the elapsed seconds of the step; loss_out and
 * logits_out (rows x dims[layers]) are optional.
 */
SYN_EXPORT double syn_baseline_mlp_step(int layers, const int *dims, int rows, const float *x,
        const int32_t *labels, float **weights, float **biases, float **m1, float **m2,
        int train, int64_t count_total, int64_t adam_step, double lr_d, double b1_d, double b2_d,
        double eps_d, float *loss_out, float *logits_out) {
    float **act = (float **)calloc((size_t)layers + 1, sizeof(float *));
    float **wt = (float **)calloc((size_t)layers, sizeof(float *));
    act[0] = (float *)x;
    size_t widest = 0;
    for (int l = 0; l <= layers; l++) if ((size_t)dims[l] > widest) widest = (size_t)dims[l];
    for (int l = 0; l < layers; l++) {
        act[l + 1] = (float *)malloc(sizeof(float) * (size_t)rows * (size_t)dims[l + 1]);
        wt[l] = (float *)malloc(sizeof(float) * (size_t)dims[l] * (size_t)dims[l + 1]);
    }
    float *dz = NULL, *da = NULL, *xt = NULL, *dwt = NULL, *dw = NULL, *db = NULL;
    double *row_loss = NULL;
    if (train) {
        dz = (float *)malloc(sizeof(float) * (size_t)rows * widest);
        da = (float *)malloc(sizeof(float) * (size_t)rows * widest);
        xt = (float *)malloc(sizeof(float) * (size_t)rows * widest);
        dwt = (float *)malloc(sizeof(float) * widest * widest);
        dw = (float *)malloc(sizeof(float) * widest * widest);
        db = (float *)malloc(sizeof(float) * widest);
        row_loss = (double *)malloc(sizeof(double) * (size_t)rows);
    }
    double t0 = now_seconds();
    /* forward: PERMUTE view copied dense, MATMUL, ADD bias, RELU */
    for (int l = 0; l < layers; l++) {
        int k = dims[l], n = dims[l + 1];
        transpose_copy(n, k, weights[l], wt[l]);
        gemm_nn(rows, n, k, act[l], wt[l], act[l + 1]);
        bias_ctx bc = {n, l + 1 < layers, act[l + 1], biases[l]};
        parallel_range(rows, bias_rows, &bc);
    }
    int classes = dims[layers];
    if (logits_out) memcpy(logits_out, act[layers], sizeof(float) * (size_t)rows * (size_t)classes);
    if (train) {
        ce_ctx cc = {classes, act[layers], labels, dz, 1.0f / (float)count_total, row_loss};
        parallel_range(rows, ce_rows, &cc);
        float loss_sum = 0.0f;
        for (int i = 0; i < rows; i++) loss_sum += (float)row_loss[i];
        if (loss_out) *loss_out = loss_sum / (float)rows;
        float c1 = 1.0f - (float)pow((double)(float)b1_d, (double)adam_step);
        float c2 = 1.0f - (float)pow((double)(float)b2_d, (double)adam_step);
        for (int l = layers - 1; l >= 0; l--) {
            int k = dims[l], n = dims[l + 1];
            colsum_ctx sc = {rows, n, dz, db};                 /* db = SUM_TO_SHAPE(dz) */
            parallel_range(n, colsum_cols, &sc);
            /* dWt[K,N] = Xt[K,M] . dz[M,N]; then PERMUTE back to [N,K] */
            transpose_copy(rows, k, act[l], xt);
            gemm_nn(k, n, rows, xt, dz, dwt);
            transpose_copy(k, n, dwt, dw);
            if (l > 0) {
                /* dA = dz[M,N] . W[N,K], then WHERE(z > 0, dA, 0) */
                gemm_nn(rows, k, n, dz, weights[l], da);
                mask_ctx mc = {act[l], da};
                parallel_range((int64_t)rows * k, mask_range, &mc);
            }
            for (int which = 0; which < 2; which++) {          /* Adam on weight then bias */
                adam_ctx ac = {which ? biases[l] : weights[l], m1[2 * l + which], m2[2 * l + which],
                               which ? db : dw, (float)lr_d, (float)b1_d, (float)b2_d, (float)eps_d, c1, c2};
                parallel_range(which ? (int64_t)n : (int64_t)n * k, adam_range, &ac);
            }
            float *swap = dz; dz = da; da = swap;
        }
    }
    double elapsed = now_seconds() - t0;
    for (int l = 0; l < layers; l++) { free(act[l + 1]); free(wt[l]); }
    free(act); free(wt); free(dz); free(da); free(xt); free(dwt); free(dw); free(db); free(row_loss);
    return elapsed;
}
