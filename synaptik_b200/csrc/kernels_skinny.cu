// Streaming CUDA-core kernels for products with one extent of at most 16 (the 10-class head of the
// classifier: forward, weight gradient and input gradient).  Such products read or write a
// [rows, 4096] activation once and do ten multiply-adds per element, so they are bounded by HBM,
// not by arithmetic: no tensor cores, 128-bit coalesced accesses, operands that are reused kept in
// registers or shared memory.
#include "kernels.hpp"

namespace syn {
namespace kern {

namespace {

__device__ __forceinline__ float relu_value(float x) { return x != x ? x : (x > 0.0f ? x : 0.0f); }

// ---- narrow result: C[m, N] = A[m, k] . W[N, k]^T (+ bias, ReLU) ---------------------------------
// W (N x k floats) is staged once per block in shared memory; a warp takes four rows at a time,
// lanes stride over k with float4 loads, and the 4 x N partial sums are combined by shuffles.
template <int N>
__global__ void __launch_bounds__(512, 1) narrow_out_kernel(int64_t m, int k, const float *__restrict__ a, int64_t lda,
        const float *__restrict__ w, int64_t ldw, const float *__restrict__ bias, int relu, float *c, int64_t c_ms, int64_t c_ns) {
    extern __shared__ float ws[];
    for (int i = threadIdx.x * 4; i < N * k; i += blockDim.x * 4) {
        int n = i / k, kk = i - n * k;
        *reinterpret_cast<float4 *>(ws + i) = *reinterpret_cast<const float4 *>(w + (int64_t)n * ldw + kk);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r0 = warp * 4; r0 < m; r0 += warps * 4) {
        float acc[4][N];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int n = 0; n < N; n++) acc[r][n] = 0.0f;
        const float *rows[4];
#pragma unroll
        for (int r = 0; r < 4; r++) rows[r] = a + (r0 + r < m ? r0 + r : m - 1) * lda;
#pragma unroll 2
        for (int kk = lane * 4; kk < k; kk += 128) {
            float4 x[4];
#pragma unroll
            for (int r = 0; r < 4; r++) x[r] = *reinterpret_cast<const float4 *>(rows[r] + kk);
#pragma unroll
            for (int n = 0; n < N; n++) {
                const float4 wv = *reinterpret_cast<const float4 *>(ws + n * k + kk);
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    acc[r][n] = fmaf(x[r].x, wv.x, acc[r][n]);
                    acc[r][n] = fmaf(x[r].y, wv.y, acc[r][n]);
                    acc[r][n] = fmaf(x[r].z, wv.z, acc[r][n]);
                    acc[r][n] = fmaf(x[r].w, wv.w, acc[r][n]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int n = 0; n < N; n++) {
                float v = acc[r][n];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
                if (lane == ((r * N + n) & 31) && r0 + r < m) {
                    if (bias) v = __fadd_rn(v, bias[n]);
                    c[(r0 + r) * c_ms + n * c_ns] = relu ? relu_value(v) : v;
                }
            }
    }
}

// ---- narrow contraction: C[m, n] = A[m, K] . B[K, n], optionally gated (ReLU backward) -----------
// A warp owns 128 consecutive result columns and keeps its K x 4 slice of B in registers; it then
// streams rows: K broadcast loads of A, one gate load and one store per row.  Every cell is the
// reference's ascending-k chain of separately rounded multiply and add, so the result is
// bit-identical to the exact kernel.
template <int K>
__global__ void __launch_bounds__(256) narrow_inner_kernel(int64_t m, int64_t n, const float *__restrict__ a, int64_t lda,
        const float *__restrict__ b, int64_t ldb, const float *__restrict__ gate, float *c, int64_t ldc, int strips) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int strip = (int)(warp % strips);
    const int64_t first = warp / strips, step = warps / strips;
    if (first >= step) return;                         // warps beyond a whole number of strip groups idle
    const int64_t col = (int64_t)strip * 128 + lane * 4;
    if (col >= n) return;
    float4 w[K];
#pragma unroll
    for (int p = 0; p < K; p++) w[p] = *reinterpret_cast<const float4 *>(b + p * ldb + col);
    // Four rows per trip, all their loads issued before the arithmetic: with one row in flight per
    // warp the kernel waited on memory latency (measured 2.2 TB/s of result + gate traffic).
    constexpr int ROWS = 4;
    for (int64_t r = first; r < m; r += step * ROWS) {
        float sv[ROWS][K];
        float4 g[ROWS];
#pragma unroll
        for (int q = 0; q < ROWS; q++) {
            const int64_t rr = r + q * step;
            const bool live = rr < m;
#pragma unroll
            for (int p = 0; p < K; p++) sv[q][p] = live ? __ldg(a + rr * lda + p) : 0.0f;
            g[q] = (gate && live) ? *reinterpret_cast<const float4 *>(gate + rr * n + col) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        }
#pragma unroll
        for (int q = 0; q < ROWS; q++) {
            const int64_t rr = r + q * step;
            if (rr >= m) break;
            float4 acc;
            if (K == 1) {
                acc = make_float4(__fmul_rn(sv[q][0], w[0].x), __fmul_rn(sv[q][0], w[0].y), __fmul_rn(sv[q][0], w[0].z), __fmul_rn(sv[q][0], w[0].w));
            } else {
                acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int p = 0; p < K; p++) {
                    const float sc = sv[q][p];
                    acc.x = __fadd_rn(acc.x, __fmul_rn(sc, w[p].x));
                    acc.y = __fadd_rn(acc.y, __fmul_rn(sc, w[p].y));
                    acc.z = __fadd_rn(acc.z, __fmul_rn(sc, w[p].z));
                    acc.w = __fadd_rn(acc.w, __fmul_rn(sc, w[p].w));
                }
            }
            if (gate) {
                acc.x = g[q].x > 0.0f ? acc.x : 0.0f; acc.y = g[q].y > 0.0f ? acc.y : 0.0f;
                acc.z = g[q].z > 0.0f ? acc.z : 0.0f; acc.w = g[q].w > 0.0f ? acc.w : 0.0f;
            }
            *reinterpret_cast<float4 *>(c + rr * ldc + col) = acc;
        }
    }
}

// ---- narrow weight gradient: D[i, j] = sum_r S[r, i] * T[r, j], i over a wide axis, j < N ----------
// Phase 1: a block owns one slice of the long axis r and eight strips of 128 consecutive i (one per
// warp).  The slice's rows of T (N floats each) are staged in shared memory 128 rows at a time, so the
// inner loop issues one 16-byte load of S per row and reads T as shared-memory broadcasts; each warp
// keeps N float4 sums in registers and streams its rows of S once.  Phase 2 adds the slices in a
// fixed order.
constexpr int kReduceChunk = 128;
template <int N>
__global__ void __launch_bounds__(256) narrow_reduce_partial_kernel(int64_t wide, int64_t depth, const float *__restrict__ s, int64_t lds,
        const float *__restrict__ t, int64_t ldt, float *partial, int strip_groups, int64_t rows_per, int64_t slices) {
    __shared__ float tchunk[kReduceChunk][N];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t slice = blockIdx.x / strip_groups;
    const int strip = (int)(blockIdx.x % strip_groups) * 8 + w;
    const int64_t col = (int64_t)strip * 128 + lane * 4;
    const int64_t r0 = slice * rows_per, r1 = r0 + rows_per < depth ? r0 + rows_per : depth;
    const bool live = col < wide;                        // a slice without rows still writes its zeros
    float4 acc[N];
#pragma unroll
    for (int j = 0; j < N; j++) acc[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    for (int64_t c0 = r0; c0 < r1; c0 += kReduceChunk) {
        const int rows_here = (int)(r1 - c0 < kReduceChunk ? r1 - c0 : kReduceChunk);
        __syncthreads();                                 // the previous chunk has been consumed
        for (int e = threadIdx.x; e < rows_here * N; e += blockDim.x) {
            const int rr = e / N, j = e - rr * N;
            tchunk[rr][j] = __ldg(t + (c0 + rr) * ldt + j);
        }
        __syncthreads();
        if (live) {
#pragma unroll 4
            for (int rr = 0; rr < rows_here; rr++) {
                const float4 sv = *reinterpret_cast<const float4 *>(s + (c0 + rr) * lds + col);
#pragma unroll
                for (int j = 0; j < N; j++) {
                    const float tv = tchunk[rr][j];
                    acc[j].x = fmaf(sv.x, tv, acc[j].x); acc[j].y = fmaf(sv.y, tv, acc[j].y);
                    acc[j].z = fmaf(sv.z, tv, acc[j].z); acc[j].w = fmaf(sv.w, tv, acc[j].w);
                }
            }
        }
    }
    if (live) {
#pragma unroll
        for (int j = 0; j < N; j++) *reinterpret_cast<float4 *>(partial + (slice * N + j) * wide + col) = acc[j];
    }
}

__global__ void narrow_reduce_final_kernel(int64_t wide, int n, int64_t slices, const float *__restrict__ partial,
                                           float *out, int64_t stride_wide, int64_t stride_narrow) {
    const int64_t total = wide * n;
    for (int64_t e = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
        const int64_t j = e / wide, i = e - j * wide;
        float sum = 0.0f;
        for (int64_t sl = 0; sl < slices; sl++) sum += partial[(sl * n + j) * wide + i];
        out[i * stride_wide + j * stride_narrow] = sum;
    }
}

constexpr int kNarrowWarps = 148 * 16;

template <template <int> class Launcher, typename... Args>
bool dispatch_extent(int extent, Args... args) {
    switch (extent) {
#define SYN_CASE(V) case V: Launcher<V>::run(args...); return true;
        SYN_CASE(1) SYN_CASE(2) SYN_CASE(3) SYN_CASE(4) SYN_CASE(5) SYN_CASE(6) SYN_CASE(7) SYN_CASE(8)
        SYN_CASE(9) SYN_CASE(10) SYN_CASE(11) SYN_CASE(12) SYN_CASE(13) SYN_CASE(14) SYN_CASE(15) SYN_CASE(16)
#undef SYN_CASE
    }
    return false;
}

template <int N> struct LaunchOut {
    static void run(cudaStream_t s, int blocks, size_t smem, int64_t m, int k, const float *a, int64_t lda, const float *w, int64_t ldw,
                    const float *bias, int relu, float *c, int64_t c_ms, int64_t c_ns) {
        cudaFuncSetAttribute(narrow_out_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        narrow_out_kernel<N><<<blocks, 512, smem, s>>>(m, k, a, lda, w, ldw, bias, relu, c, c_ms, c_ns);
    }
};
template <int K> struct LaunchInner {
    static void run(cudaStream_t s, int blocks, int64_t m, int64_t n, const float *a, int64_t lda, const float *b, int64_t ldb,
                    const float *gate, float *c, int64_t ldc, int strips) {
        narrow_inner_kernel<K><<<blocks, 256, 0, s>>>(m, n, a, lda, b, ldb, gate, c, ldc, strips);
    }
};
template <int N> struct LaunchReduce {
    static void run(cudaStream_t s, int blocks, int64_t wide, int64_t depth, const float *src, int64_t lds, const float *t, int64_t ldt,
                    float *partial, int strip_groups, int64_t rows_per, int64_t slices) {
        narrow_reduce_partial_kernel<N><<<blocks, 256, 0, s>>>(wide, depth, src, lds, t, ldt, partial, strip_groups, rows_per, slices);
    }
};

inline bool aligned16(const void *p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace

bool narrow_out_supported(int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldw) {
    return n >= 1 && n <= 16 && m >= 1 && k >= 128 && (k & 3) == 0 && (lda & 3) == 0 && (ldw & 3) == 0 && n * k * 4 <= 200 * 1024 && k < (1 << 30);
}

cudaError_t gemm_narrow_out(cudaStream_t s, int sm_count, int64_t m, int64_t n, int64_t k, const float *a, int64_t lda,
                            const float *w, int64_t ldw, const float *bias, int relu, float *c, int64_t c_ms, int64_t c_ns) {
    if (!narrow_out_supported(m, n, k, lda, ldw) || !aligned16(a) || !aligned16(w)) return cudaErrorInvalidValue;
    size_t smem = (size_t)n * k * 4;
    int64_t groups = (m + 3) / 4, blocks = (groups + 15) / 16;
    if (blocks > sm_count) blocks = sm_count;
    dispatch_extent<LaunchOut>((int)n, s, (int)blocks, smem, m, (int)k, a, lda, w, ldw, bias, relu, c, c_ms, c_ns);
    return cudaGetLastError();
}

bool narrow_inner_supported(int64_t m, int64_t n, int64_t k, int64_t ldb, int64_t ldc) {
    return k >= 1 && k <= 16 && m >= 1 && n >= 128 && (n & 3) == 0 && (ldb & 3) == 0 && (ldc & 3) == 0;
}

cudaError_t gemm_narrow_inner(cudaStream_t s, int64_t m, int64_t n, int64_t k, const float *a, int64_t lda,
                              const float *b, int64_t ldb, const float *gate, float *c, int64_t ldc) {
    if (!narrow_inner_supported(m, n, k, ldb, ldc) || !aligned16(b) || !aligned16(c) || (gate && !aligned16(gate))) return cudaErrorInvalidValue;
    int strips = (int)((n + 127) / 128);
    int64_t groups = kNarrowWarps / strips;
    if (groups < 1) groups = 1;
    if (groups > m) groups = m;
    int64_t warps = groups * strips;
    int blocks = (int)((warps + 7) / 8);
    dispatch_extent<LaunchInner>((int)k, s, blocks, m, n, a, lda, b, ldb, gate, c, ldc, strips);
    return cudaGetLastError();
}

bool narrow_reduce_supported(int64_t wide, int64_t n, int64_t depth, int64_t lds) {
    return n >= 1 && n <= 16 && wide >= 128 && (wide & 3) == 0 && (lds & 3) == 0 && depth >= 1;
}

static int64_t narrow_reduce_slices(int64_t wide, int64_t depth) {
    int64_t strips = (wide + 127) / 128;
    int64_t slices = kNarrowWarps / strips;
    int64_t most = (depth + 63) / 64;
    if (slices > most) slices = most;
    return slices < 1 ? 1 : slices;
}

int64_t narrow_reduce_partial_floats(int64_t wide, int64_t n, int64_t depth) { return narrow_reduce_slices(wide, depth) * n * wide; }

cudaError_t gemm_narrow_reduce(cudaStream_t s, int64_t wide, int64_t n, int64_t depth, const float *src, int64_t lds,
                               const float *t, int64_t ldt, float *partial, float *out, int64_t stride_wide, int64_t stride_narrow) {
    if (!narrow_reduce_supported(wide, n, depth, lds) || !aligned16(src) || !aligned16(partial)) return cudaErrorInvalidValue;
    int strips = (int)((wide + 127) / 128);
    int strip_groups = (strips + 7) / 8;
    int64_t slices = narrow_reduce_slices(wide, depth);
    int64_t rows_per = (depth + slices - 1) / slices;
    int blocks = (int)(slices * strip_groups);
    dispatch_extent<LaunchReduce>((int)n, s, blocks, wide, depth, src, lds, t, ldt, partial, strip_groups, rows_per, slices);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    int64_t total = wide * n;
    narrow_reduce_final_kernel<<<(unsigned)((total + 255) / 256 > 1184 ? 1184 : (total + 255) / 256), 256, 0, s>>>(wide, (int)n, slices, partial, out, stride_wide, stride_narrow);
    return cudaGetLastError();
}

}  // namespace kern
}  // namespace syn
