// Memory-bound kernels of the dense-MLP path: node-by-node elementwise operations, row
// reductions, softmax / cross-entropy / arg-max row kernels, column sums, and the fused optimizer
// passes.  All use coalesced (128-bit where alignment allows) accesses and warp-shuffle
// reductions; none uses tensor cores on purpose -- they are bounded by HBM bandwidth.
#include "kernels.hpp"
#include "activation.cuh"
#include "lowp.cuh"
#include "split.cuh"

#include <cfloat>
#include <math_constants.h>
#include <cmath>
#include <mutex>

namespace syn {
namespace kern {

namespace {

constexpr int kThreads = 256;

inline int grid_for(int64_t total, int per_block, int cap = 148 * 16) {
    int64_t blocks = (total + per_block - 1) / per_block;
    if (blocks < 1) blocks = 1;
    return (int)(blocks > cap ? cap : blocks);
}

// exp(x) in binary32, within 0.78 ulp of the exact value (measured on the host over a uniform
// sweep of bit patterns) and equal to the correctly rounded value for 99.7 % of inputs; the
// reference computes (float)StrictMath.exp((double)x).  Cody-Waite reduction by ln2 in two parts,
// degree-7 polynomial, compensated final addition, two-step power-of-two scaling so subnormal
// results round once.
__device__ __forceinline__ float exp_accurate(float x) {
    if (!(x > -104.0f)) return x != x ? x : 0.0f;
    if (x > 88.8f) return __int_as_float(0x7f800000);
    float n = rintf(x * 1.4426950408889634f);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.42860682030941723212e-6f, r);
    float p = 1.9841270114e-4f;
    p = fmaf(p, r, 1.3888889225e-3f);
    p = fmaf(p, r, 8.3333337680e-3f);
    p = fmaf(p, r, 4.1666667908e-2f);
    p = fmaf(p, r, 1.6666667163e-1f);
    p = fmaf(p, r, 0.5f);
    float t = __fmul_rn(__fmul_rn(r, r), p);
    float s = __fadd_rn(1.0f, r);
    float err = __fadd_rn(__fsub_rn(1.0f, s), r);
    float res = __fadd_rn(s, __fadd_rn(err, t));
    int ni = (int)n;
    int n1 = ni < -126 ? -126 : (ni > 127 ? 127 : ni);
    int n2 = ni - n1;
    return __fmul_rn(__fmul_rn(res, __int_as_float((n1 + 127) << 23)), __int_as_float((n2 + 127) << 23));
}

// exp(x) for finite x <= 0 (logits shifted by their row maximum), the hot form inside the row
// kernels: same reduction and polynomial as exp_accurate, rounding to the nearest integer by the
// 1.5 * 2^23 trick, scaling by a power of two assembled in the exponent field.  Within 1.03 ulp,
// equal to the correctly rounded value for 99.2 % of inputs (host sweep).  Arguments below -87.33
// are clamped there, so results that would be subnormal come out as 1.18e-38: an absolute error
// below 1.2e-38 next to a row maximum whose exponential is 1.  NaN and infinities are not handled
// here: rows that contain them take the careful path.
__device__ __forceinline__ float exp_shifted(float x) {
    const float magic = 12582912.0f;
    x = fmaxf(x, -87.33f);
    float t = fmaf(x, 1.4426950408889634f, magic);
    float n = __fsub_rn(t, magic);
    float r = fmaf(n, -0.693145751953125f, x);
    r = fmaf(n, -1.42860682030941723212e-6f, r);
    float q = 1.9841270114e-4f;
    q = fmaf(q, r, 1.3888889225e-3f);
    q = fmaf(q, r, 8.3333337680e-3f);
    q = fmaf(q, r, 4.1666667908e-2f);
    q = fmaf(q, r, 1.6666667163e-1f);
    q = fmaf(q, r, 0.5f);
    float res = __fadd_rn(fmaf(__fmul_rn(r, r), q, r), 1.0f);
    // scaling by 2^n in the exponent field: the low bits of t hold n (the magic constant's own bits
    // shift out), and res * 2^n stays normal because the clamp keeps n >= -126 with res >= 1 there
    return __int_as_float(__float_as_int(res) + (__float_as_int(t) << 23));
}

__device__ __forceinline__ float java_max(float a, float b) {   // Math.max: NaN wins, +0 above -0
    if (a != a) return a;
    if (b != b) return b;
    if (a == 0.0f && b == 0.0f) return (__float_as_uint(a) >> 31) ? b : a;
    return a > b ? a : b;
}

__device__ __forceinline__ float java_min(float a, float b) {   // Math.min: NaN wins, -0 below +0
    if (a != a) return a;
    if (b != b) return b;
    if (a == 0.0f && b == 0.0f) return (__float_as_uint(a) >> 31) ? a : b;
    return a < b ? a : b;
}

__device__ __forceinline__ double warp_sum(double v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max_java(float v) {
    for (int o = 16; o > 0; o >>= 1) v = java_max(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_max_plain(float v) {     // the plain '>' maximum of logSumExp
    for (int o = 16; o > 0; o >>= 1) { float u = __shfl_xor_sync(0xffffffffu, v, o); v = u > v ? u : v; }
    return v;
}

__device__ __forceinline__ void unravel(int64_t i, const Index4 &ix, int64_t &oa, int64_t &ob, int64_t &oc) {
    int64_t i3 = i % ix.shape[3]; i /= ix.shape[3];
    int64_t i2 = i % ix.shape[2]; i /= ix.shape[2];
    int64_t i1 = i % ix.shape[1]; int64_t i0 = i / ix.shape[1];
    oa = i0 * ix.sa[0] + i1 * ix.sa[1] + i2 * ix.sa[2] + i3 * ix.sa[3];
    ob = i0 * ix.sb[0] + i1 * ix.sb[1] + i2 * ix.sb[2] + i3 * ix.sb[3];
    oc = i0 * ix.sc[0] + i1 * ix.sc[1] + i2 * ix.sc[2] + i3 * ix.sc[3];
}

template <typename T> struct UnsignedOf;
template <> struct UnsignedOf<int32_t> { typedef uint32_t type; };
template <> struct UnsignedOf<int64_t> { typedef uint64_t type; };

__global__ void binary_kernel(int op, const float *__restrict__ a, const float *__restrict__ b, void *out, Index4 ix, int64_t total) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t oa, ob, oc;
        unravel(i, ix, oa, ob, oc);
        float x = a[oa], y = b[ob];
        switch ((Op)op) {
            case Op::ADD: ((float *)out)[i] = __fadd_rn(x, y); break;
            case Op::SUB: ((float *)out)[i] = __fsub_rn(x, y); break;
            case Op::MUL: ((float *)out)[i] = __fmul_rn(x, y); break;
            case Op::DIV: ((float *)out)[i] = __fdiv_rn(x, y); break;
            case Op::LT: ((uint8_t *)out)[i] = x < y ? 1 : 0; break;
            case Op::EQ: ((uint8_t *)out)[i] = x == y ? 1 : 0; break;
            default: ((uint8_t *)out)[i] = x > y ? 1 : 0; break;          // GT
        }
    }
}

// Integer operands: SUB wraps like Java's int / long arithmetic, EQ compares exactly.  The index
// cross-entropy gradient rule tests labels against the ignore index with these
// (LossGradientRules.java:203-207).
template <typename T>
__global__ void binary_int_kernel(int op, const T *__restrict__ a, const T *__restrict__ b, void *out, Index4 ix, int64_t total) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t oa, ob, oc;
        unravel(i, ix, oa, ob, oc);
        T x = a[oa], y = b[ob];
        if ((Op)op == Op::SUB) ((T *)out)[i] = (T)((typename UnsignedOf<T>::type)x - (typename UnsignedOf<T>::type)y);
        else ((uint8_t *)out)[i] = x == y ? 1 : 0;
    }
}

__global__ void where_kernel(const uint8_t *__restrict__ cond, const float *__restrict__ a, const float *__restrict__ b,
                             float *out, Index4 ix, int64_t total) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t oc, oa, ob;
        unravel(i, ix, oc, oa, ob);      // strides: sa = condition, sb = first, sc = second
        out[i] = cond[oc] ? a[oa] : b[ob];
    }
}

template <typename T>
__global__ void scalar_kernel(int op, const T *__restrict__ a, T *out, T scalar, int64_t total) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        T x = a[i];
        if ((Op)op == Op::SCALAR_MIN) out[i] = x < scalar ? x : scalar;
        else if ((Op)op == Op::SCALAR_SUB) out[i] = (T)((typename UnsignedOf<T>::type)x - (typename UnsignedOf<T>::type)scalar);   // wraps like Java
        else out[i] = x > scalar ? x : scalar;
    }
}
__global__ void scalar_f32_kernel(int op, const float *__restrict__ a, float *out, float scalar, int64_t total) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float x = a[i];
        if ((Op)op == Op::SCALAR_MUL) out[i] = __fmul_rn(x, scalar);
        else if ((Op)op == Op::SCALAR_SUB) out[i] = __fsub_rn(x, scalar);
        else if ((Op)op == Op::SCALAR_MIN) out[i] = java_min(x, scalar);
        else out[i] = java_max(x, scalar);
    }
}

__global__ void unary_kernel(int op, const float *__restrict__ a, void *out_raw, int64_t total) {
    float *out = static_cast<float *>(out_raw);
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        float x = a[i];
        switch ((Op)op) {
            case Op::RELU: out[i] = relu_value(x); break;
            case Op::TANH: out[i] = tanh_value(x); break;
            case Op::SIGMOID: out[i] = sigmoid_value(x); break;
            case Op::SILU: out[i] = silu_value(x); break;
            case Op::GELU_TANH: out[i] = gelu_tanh_value(x); break;
            case Op::GELU: out[i] = gelu_value(x); break;
            case Op::ERF: out[i] = erf_value(x); break;
            case Op::IS_INF: static_cast<uint8_t *>(out_raw)[i] = (__float_as_uint(x) & 0x7fffffffu) == 0x7f800000u; break;
            default: out[i] = exp_accurate(x); break;
        }
    }
}

template <typename T>
__global__ void one_hot_kernel(const T *__restrict__ indices, uint8_t *out, int64_t count, int64_t depth) {
    int64_t total = count * depth;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t row = i / depth, col = i - row * depth;
        out[i] = (int64_t)indices[row] == col ? 1 : 0;
    }
}

template <typename T>
__global__ void copy_kernel(const T *__restrict__ src, T *dst, Index4 ix, int64_t total) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t oa, ob, oc;
        unravel(i, ix, oa, ob, oc);
        dst[i] = src[oa];
    }
}

// One warp per row.  SUM accumulates in binary64 and rounds once (the reference's aggregate SUM is
// exactly rounded, CpuExactSumEmitter.java:14-21); MAX follows Math.max.
__global__ void row_reduce_kernel(int op, const float *__restrict__ x, float *out, int64_t rows, int64_t cols) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += warps) {
        const float *row = x + r * cols;
        if ((Op)op == Op::SUM) {
            double acc = 0.0;
            for (int64_t c = lane; c < cols; c += 32) acc += (double)row[c];
            acc = warp_sum(acc);
            if (lane == 0) out[r] = (float)acc;
        } else {
            float acc = row[0];
            for (int64_t c = lane; c < cols; c += 32) acc = java_max(acc, row[c]);
            acc = warp_max_java(acc);
            if (lane == 0) out[r] = acc;
        }
    }
}

__global__ void full_sum_kernel(const float *__restrict__ x, Index4 ix, int64_t total, float *out) {
    __shared__ double partial[32];
    double acc = 0.0;
    for (int64_t i = threadIdx.x; i < total; i += blockDim.x) {
        int64_t oa, ob, oc;
        unravel(i, ix, oa, ob, oc);
        acc += (double)x[oa];
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        double v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.0;
        v = warp_sum(v);
        if (threadIdx.x == 0) out[0] = (float)v;
    }
}

// Total order key of ARG_MAX (CpuArgExtremaEmitter.java:268-318): every NaN above +inf, -0 below +0.
__device__ __forceinline__ uint32_t order_key(float v) {
    uint32_t b = __float_as_uint(v);
    if ((b & 0x7fffffffu) > 0x7f800000u) return 0xffffffffu;
    return (b >> 31) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long warp_best(unsigned long long v) {
    for (int o = 16; o > 0; o >>= 1) { unsigned long long u = __shfl_xor_sync(0xffffffffu, v, o); v = u > v ? u : v; }
    return v;
}

__device__ __forceinline__ uint32_t warp_umin(uint32_t v) {
    for (int o = 16; o > 0; o >>= 1) { uint32_t u = __shfl_xor_sync(0xffffffffu, v, o); v = u < v ? u : v; }
    return v;
}

// Row arg-max of a row held in registers (lane l holds float4 chunks l, l+32, ...).  Common rows
// (no NaN, maximum not a zero) take the cheap route: plain maximum, then the first column equal to
// it.  Rows with a NaN or a zero maximum take the total-order key so that NaN wins and -0 < +0.
template <int CHUNKS>
__device__ __forceinline__ int64_t warp_row_argmax(const float4 (&v)[CHUNKS], int vec_cols, int lane) {
    // groups past the row's end hold -FLT_MAX (the caller pads): they never win and never flag
    float m = __int_as_float(0xff800000), probe = 0.0f;
    float m4[CHUNKS];                       // maximum of each 16-byte group
#pragma unroll
    for (int j = 0; j < CHUNKS; j++) {
        m4[j] = fmaxf(fmaxf(v[j].x, v[j].y), fmaxf(v[j].z, v[j].w));
        m = fmaxf(m, m4[j]);
        // x * 0 accumulates on the FMA pipe and turns NaN for any NaN or infinity in the row
        probe = fmaf(v[j].x, 0.0f, probe); probe = fmaf(v[j].y, 0.0f, probe);
        probe = fmaf(v[j].z, 0.0f, probe); probe = fmaf(v[j].w, 0.0f, probe);
    }
    m = warp_max_plain(m);
    if (!__any_sync(0xffffffffu, probe != probe) && m != 0.0f) {
        // finite row, non-zero maximum: the first column equal to it; only a group whose own maximum
        // is the row maximum is looked into
        uint32_t first = 0xffffffffu;
#pragma unroll
        for (int j = CHUNKS - 1; j >= 0; j--) {
            if (m4[j] == m) {
                const uint32_t c4 = (uint32_t)(lane + 32 * j) * 4;
                first = v[j].w == m ? c4 + 3 : first;
                first = v[j].z == m ? c4 + 2 : first;
                first = v[j].y == m ? c4 + 1 : first;
                first = v[j].x == m ? c4 : first;
            }
        }
        return (int64_t)warp_umin(first);
    }
    unsigned long long best = 0;
#pragma unroll
    for (int j = 0; j < CHUNKS; j++) {
        const int c = lane + 32 * j;
        if (c < vec_cols) {
            const float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                unsigned long long cand = ((unsigned long long)order_key(e[q]) << 32) | (0xffffffffu - (uint32_t)(c * 4 + q));
                best = cand > best ? cand : best;
            }
        }
    }
    best = warp_best(best);
    return (int64_t)(0xffffffffu - (uint32_t)(best & 0xffffffffu));
}

template <int CHUNKS>
__global__ void __launch_bounds__(kThreads) argmax_vec_kernel(const float *__restrict__ x, int64_t *out, int64_t rows, int cols) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int vec_cols = cols >> 2;
    for (int64_t r = warp; r < rows; r += warps) {
        const float4 *row = reinterpret_cast<const float4 *>(x + r * cols);
        float4 v[CHUNKS];
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) v[j] = lane + 32 * j < vec_cols ? row[lane + 32 * j] : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        // the row this warp takes next, asked into L2 meanwhile (one 128-byte line per lane)
        if (r + warps < rows && lane * 32 < cols)
            asm volatile("prefetch.global.L2 [%0];" :: "l"(x + (r + warps) * cols + lane * 32));
        int64_t best = warp_row_argmax<CHUNKS>(v, vec_cols, lane);
        if (lane == 0) out[r] = best;
    }
}

__global__ void __launch_bounds__(kThreads) argmax_kernel(const float *__restrict__ x, int64_t *out, int64_t rows, int64_t cols) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += warps) {
        const float *row = x + r * cols;
        // larger key wins; among equal keys the smaller index wins (FIRST_INDEX ties)
        unsigned long long best = 0;
        for (int64_t c = lane; c < cols; c += 32) {
            unsigned long long cand = ((unsigned long long)order_key(row[c]) << 32) | (0xffffffffu - (uint32_t)c);
            best = cand > best ? cand : best;
        }
        best = warp_best(best);
        if (lane == 0) out[r] = (int64_t)(0xffffffffu - (uint32_t)(best & 0xffffffffu));
    }
}

// SOFTMAX / LOG_SOFTMAX rows, CpuSoftmaxReferenceKernel.java:104-146: Math.max maximum; any +inf ->
// NaN at the infinities and 0 (LOG_SOFTMAX: -inf) elsewhere; any -inf (without NaN) -> unshifted
// exponentials; otherwise exp(x - max) / sum, or (x - max) - (float)log(sum) for LOG_SOFTMAX (the
// logarithm of the sum, never of the rounded quotient, so a far-away column keeps its finite
// distance).  The reference's Kahan-compensated binary32 sum is replaced by a binary64 sum
// rounded once (both lie within an ulp of the exact sum).
// One row, any values and any width (three passes over the row in memory).
template <bool LOG>
__device__ __forceinline__ void softmax_row_careful(const float *__restrict__ row, float *o, int64_t cols, int lane) {
    float maximum = __int_as_float(0xff800000);
    int has_ninf = 0;
    for (int64_t c = lane; c < cols; c += 32) { float v = row[c]; maximum = java_max(maximum, v); has_ninf |= v == __int_as_float(0xff800000); }
    maximum = warp_max_java(maximum);
    has_ninf = __any_sync(0xffffffffu, has_ninf);
    if (maximum == __int_as_float(0x7f800000)) {
        const float rest = LOG ? __int_as_float(0xff800000) : 0.0f;
        for (int64_t c = lane; c < cols; c += 32) o[c] = row[c] == maximum ? __int_as_float(0x7fc00000) : rest;
        return;
    }
    const bool unshifted = has_ninf && !(maximum != maximum);
    float sum;
    if (unshifted) {
        // a row with -inf is not shifted and the reference adds its exponentials in plain ascending
        // binary32 order, without compensation (CpuSoftmaxReferenceKernel.java:124-131): one lane follows
        // that order, since the rounding error of such a sum is part of the reference's result
        maximum = 0.0f;
        float s = 0.0f;
        if (lane == 0) for (int64_t c = 0; c < cols; c++) s = __fadd_rn(s, exp_accurate(__fsub_rn(row[c], maximum)));
        sum = __shfl_sync(0xffffffffu, s, 0);
    } else {
        double acc = 0.0;
        for (int64_t c = lane; c < cols; c += 32) acc += (double)exp_accurate(__fsub_rn(row[c], maximum));
        sum = (float)warp_sum(acc);
    }
    if (LOG) {
        const float logarithm = (float)log((double)sum);
        for (int64_t c = lane; c < cols; c += 32) o[c] = __fsub_rn(__fsub_rn(row[c], maximum), logarithm);
    } else {
        for (int64_t c = lane; c < cols; c += 32) o[c] = __fdiv_rn(exp_accurate(__fsub_rn(row[c], maximum)), sum);
    }
}

template <bool LOG>
__global__ void softmax_kernel(const float *__restrict__ x, float *out, int64_t rows, int64_t cols) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += warps) softmax_row_careful<LOG>(x + r * cols, out + r * cols, cols, lane);
}

// Rows of at most 1024 columns, 16-byte aligned: the row is read once into registers (one warp per
// row, CHUNKS 16-byte groups per lane), finite rows take the exponential once per element
// (exp_shifted, within 1.03 ulp), the row sum in binary64, and the quotient as one reciprocal per row
// plus a remainder-corrected product per element; rows with an infinity or NaN go to the careful
// routine with the reference's branches.  The next row of the warp is asked into L2 meanwhile.
template <int CHUNKS, bool LOG>
__global__ void __launch_bounds__(kThreads, CHUNKS >= 8 ? 3 : 4) softmax_rows_vec_kernel(const float *__restrict__ x, float *out, int64_t rows, int cols) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int vec_cols = cols >> 2;
    for (int64_t r = warp; r < rows; r += warps) {
        const float *row_s = x + r * cols;
        const float4 *row = reinterpret_cast<const float4 *>(row_s);
        float4 v[CHUNKS];
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) v[j] = lane + 32 * j < vec_cols ? row[lane + 32 * j] : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        if (r + warps < rows && lane * 32 < cols)
            asm volatile("prefetch.global.L2 [%0];" :: "l"(row_s + warps * cols + lane * 32));
        float maximum = __int_as_float(0xff800000), probe = 0.0f;
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            maximum = fmaxf(fmaxf(maximum, fmaxf(v[j].x, v[j].y)), fmaxf(v[j].z, v[j].w));
            probe = fmaf(v[j].x, 0.0f, probe); probe = fmaf(v[j].y, 0.0f, probe);
            probe = fmaf(v[j].z, 0.0f, probe); probe = fmaf(v[j].w, 0.0f, probe);
        }
        maximum = warp_max_plain(maximum);
        // rare: an infinity or NaN in the row, or a zero maximum whose sign reaches a LOG_SOFTMAX result
        if (__any_sync(0xffffffffu, probe != probe) || (LOG && maximum == 0.0f)) {
            softmax_row_careful<LOG>(row_s, out + r * cols, cols, lane);
            continue;
        }
        double acc = 0.0;
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            const float s0 = __fsub_rn(v[j].x, maximum), s1 = __fsub_rn(v[j].y, maximum), s2 = __fsub_rn(v[j].z, maximum), s3 = __fsub_rn(v[j].w, maximum);
            const float e0 = exp_shifted(s0), e1 = exp_shifted(s1), e2 = exp_shifted(s2), e3 = exp_shifted(s3);
            if (lane + 32 * j < vec_cols) acc += (double)__fadd_rn(__fadd_rn(e0, e1), __fadd_rn(e2, e3));
            v[j] = LOG ? make_float4(s0, s1, s2, s3) : make_float4(e0, e1, e2, e3);
        }
        const float sum = (float)warp_sum(acc);            // finite, at least 1: the maximum contributes exp(0)
        float4 *o = reinterpret_cast<float4 *>(out + r * cols);
        if (LOG) {
            const float logarithm = (float)log((double)sum);
#pragma unroll
            for (int j = 0; j < CHUNKS; j++)
                if (lane + 32 * j < vec_cols)
                    o[lane + 32 * j] = make_float4(__fsub_rn(v[j].x, logarithm), __fsub_rn(v[j].y, logarithm), __fsub_rn(v[j].z, logarithm), __fsub_rn(v[j].w, logarithm));
        } else {
            const float rcp = __frcp_rn(sum);
#pragma unroll
            for (int j = 0; j < CHUNKS; j++) {
                float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float p = __fmul_rn(e[q], rcp);
                    e[q] = fmaf(fmaf(-p, sum, e[q]), rcp, p);
                }
                if (lane + 32 * j < vec_cols) o[lane + 32 * j] = make_float4(e[0], e[1], e[2], e[3]);
            }
        }
    }
}

// Gradient node lists of SOFTMAX and LOG_SOFTMAX (ReductionGradientRules.java:84-90) in one pass per row,
// every node's rounding kept: SOFTMAX y * (g - SUM(g * y)), LOG_SOFTMAX g - exp(y) * SUM(g), the row
// SUM exactly rounded (binary64 lanes, one rounding).  One warp per row; the second sweep over the row
// comes from cache.
template <bool LOG>
__global__ void softmax_backward_rows_kernel(const float *__restrict__ y, const float *__restrict__ g, float *out, int64_t rows, int64_t cols) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const bool vec = (cols & 3) == 0 && ((((uintptr_t)y | (uintptr_t)g | (uintptr_t)out) & 15) == 0);
    for (int64_t r = warp; r < rows; r += warps) {
        const float *yr = y + r * cols, *gr = g + r * cols;
        float *o = out + r * cols;
        double acc = 0.0;
        if (vec) {
            const float4 *y4 = reinterpret_cast<const float4 *>(yr), *g4 = reinterpret_cast<const float4 *>(gr);
            for (int64_t c = lane; c < (cols >> 2); c += 32) {
                const float4 b = g4[c];
                if (LOG) acc += ((double)b.x + (double)b.y) + ((double)b.z + (double)b.w);
                else { const float4 a = y4[c]; acc += ((double)__fmul_rn(b.x, a.x) + (double)__fmul_rn(b.y, a.y)) + ((double)__fmul_rn(b.z, a.z) + (double)__fmul_rn(b.w, a.w)); }
            }
        } else {
            for (int64_t c = lane; c < cols; c += 32) acc += LOG ? (double)gr[c] : (double)__fmul_rn(gr[c], yr[c]);
        }
        const float total = (float)warp_sum(acc);
        if (vec) {
            const float4 *y4 = reinterpret_cast<const float4 *>(yr), *g4 = reinterpret_cast<const float4 *>(gr);
            float4 *o4 = reinterpret_cast<float4 *>(o);
            for (int64_t c = lane; c < (cols >> 2); c += 32) {
                const float4 a = y4[c], b = g4[c];
                float4 d;
                if (LOG) {
                    d.x = __fsub_rn(b.x, __fmul_rn(exp_accurate(a.x), total)); d.y = __fsub_rn(b.y, __fmul_rn(exp_accurate(a.y), total));
                    d.z = __fsub_rn(b.z, __fmul_rn(exp_accurate(a.z), total)); d.w = __fsub_rn(b.w, __fmul_rn(exp_accurate(a.w), total));
                } else {
                    d.x = __fmul_rn(a.x, __fsub_rn(b.x, total)); d.y = __fmul_rn(a.y, __fsub_rn(b.y, total));
                    d.z = __fmul_rn(a.z, __fsub_rn(b.z, total)); d.w = __fmul_rn(a.w, __fsub_rn(b.w, total));
                }
                o4[c] = d;
            }
        } else {
            for (int64_t c = lane; c < cols; c += 32)
                o[c] = LOG ? __fsub_rn(gr[c], __fmul_rn(exp_accurate(yr[c]), total)) : __fmul_rn(yr[c], __fsub_rn(gr[c], total));
        }
    }
}

// MEAN_SQUARED_ERROR, CpuLossReferenceKernel.java:67-87: ascending binary32 accumulation of the
// squared differences, then the exact quotient by the count rounded once (:221-225).  Small
// inputs are accumulated by one thread in the reference's order; large ones by a binary64 tree.
__global__ void squared_error_kernel(const float *__restrict__ p, const float *__restrict__ t, int64_t count, float *out) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < count; i += (int64_t)gridDim.x * blockDim.x) {
        const float d = __fsub_rn(p[i], t[i]);
        out[i] = __fmul_rn(d, d);
    }
}

__global__ void mse_kernel(const float *__restrict__ p, const float *__restrict__ t, int64_t count, float *out, int mean) {
    __shared__ double partial[32];
    float total;
    if (count <= 65536) {
        if (threadIdx.x != 0) return;
        float sum = 0.0f;
        for (int64_t i = 0; i < count; i++) { float d = __fsub_rn(p[i], t[i]); sum = __fadd_rn(sum, __fmul_rn(d, d)); }
        total = sum;
    } else {
        double acc = 0.0;
        for (int64_t i = threadIdx.x; i < count; i += blockDim.x) { float d = __fsub_rn(p[i], t[i]); acc += (double)__fmul_rn(d, d); }
        acc = warp_sum(acc);
        if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x >= 32) return;
        double v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.0;
        v = warp_sum(v);
        if (threadIdx.x != 0) return;
        total = (float)v;
    }
    // binary64 holds the quotient of a 24-bit numerator by a count below 2^28 to well under half a
    // binary32 ulp of any non-tie, so the second rounding cannot move the result
    if (!mean) { out[0] = total; return; }
    out[0] = (total == 0.0f || !isfinite(total)) ? total / (float)count : (float)((double)total / (double)count);
}

// Large inputs, two phases: every block adds its share of the squared differences in binary64 (grid-
// strided, so the order is fixed by the launch shape) and writes one partial; one block then adds the
// partials in order, rounds once and forms the quotient as above.  One block over 65 M elements took
// milliseconds; this form streams at HBM speed.
constexpr int kMsePartialThreads = 256;
__global__ void __launch_bounds__(kMsePartialThreads) mse_partial_kernel(const float *__restrict__ p, const float *__restrict__ t, int64_t count, double *partials) {
    __shared__ double partial[kMsePartialThreads / 32];
    const int64_t tid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
    double acc = 0.0;
    if ((((uintptr_t)p | (uintptr_t)t) & 15) == 0) {
        const float4 *p4 = reinterpret_cast<const float4 *>(p), *t4 = reinterpret_cast<const float4 *>(t);
        const int64_t n4 = count >> 2;
        for (int64_t i = tid; i < n4; i += stride) {
            const float4 a = p4[i], b = t4[i];
            const float d0 = __fsub_rn(a.x, b.x), d1 = __fsub_rn(a.y, b.y), d2 = __fsub_rn(a.z, b.z), d3 = __fsub_rn(a.w, b.w);
            acc += ((double)__fmul_rn(d0, d0) + (double)__fmul_rn(d1, d1)) + ((double)__fmul_rn(d2, d2) + (double)__fmul_rn(d3, d3));
        }
        for (int64_t i = (n4 << 2) + tid; i < count; i += stride) { const float d = __fsub_rn(p[i], t[i]); acc += (double)__fmul_rn(d, d); }
    } else {
        for (int64_t i = tid; i < count; i += stride) { const float d = __fsub_rn(p[i], t[i]); acc += (double)__fmul_rn(d, d); }
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double v = 0.0;
        for (int i = 0; i < kMsePartialThreads / 32; i++) v += partial[i];
        partials[blockIdx.x] = v;
    }
}

__global__ void mse_final_kernel(const double *__restrict__ partials, int blocks, int64_t count, float *out, int mean) {
    __shared__ double partial[32];
    double acc = 0.0;
    for (int i = threadIdx.x; i < blocks; i += blockDim.x) acc += partials[i];
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x >= 32) return;
    double v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.0;
    v = warp_sum(v);
    if (threadIdx.x != 0) return;
    const float total = (float)v;
    if (!mean) { out[0] = total; return; }
    out[0] = (total == 0.0f || !isfinite(total)) ? total / (float)count : (float)((double)total / (double)count);
}

__global__ void relu_backward_kernel(const float4 *__restrict__ gate, const float4 *__restrict__ up, float4 *out, int64_t vec_count,
                                     const float *gate_s, const float *up_s, float *out_s, int64_t total) {
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x, stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t v = i; v < vec_count; v += stride) {
        float4 z = gate[v], g = up[v], r;
        r.x = z.x > 0.0f ? g.x : 0.0f; r.y = z.y > 0.0f ? g.y : 0.0f;
        r.z = z.z > 0.0f ? g.z : 0.0f; r.w = z.w > 0.0f ? g.w : 0.0f;
        out[v] = r;
    }
    for (int64_t e = vec_count * 4 + i; e < total; e += stride) out_s[e] = gate_s[e] > 0.0f ? up_s[e] : 0.0f;
}

// Column sums, phase 1: block (strip, split) adds rows [split*rows_per, ...) of a 128-column strip
// in binary64 and writes one partial per column; phase 2 adds the partials of each column in a
// fixed order and rounds once.  Deterministic, no atomics.
constexpr int kColsumRows = 8;     // warps per block, each striding over rows
// PLANES: the pass also writes the hi / lo operand planes (row pitch `pitch`) of the matrix it reads,
// so a gradient that is both summed over rows (bias gradient) and fed to tensor-core products is read
// from HBM once for both.
template <bool PLANES>
__global__ void colsum_partial_kernel(const float *__restrict__ g, int64_t rows, int64_t cols, int64_t rows_per, double *partials,
                                      float *hi, float *lo, int64_t pitch) {
    __shared__ double sm[kColsumRows][128];
    int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    int64_t col0 = (int64_t)blockIdx.x * 128 + lane * 4;
    int64_t r0 = (int64_t)blockIdx.y * rows_per, r1 = r0 + rows_per < rows ? r0 + rows_per : rows;
    double a0 = 0, a1 = 0, a2 = 0, a3 = 0;
    bool vec = (cols & 3) == 0 && col0 + 3 < cols && ((uintptr_t)g & 15) == 0;
    if (vec) {
        // four rows per trip, their loads issued together: one row in flight per warp left the pass
        // latency-bound once it also wrote the planes
        int64_t r = r0 + w;
        for (; r + 3 * kColsumRows < r1; r += 4 * kColsumRows) {
            float4 v[4];
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = *reinterpret_cast<const float4 *>(g + (r + q * kColsumRows) * cols + col0);
#pragma unroll
            for (int q = 0; q < 4; q++) {
                a0 += v[q].x; a1 += v[q].y; a2 += v[q].z; a3 += v[q].w;
                if (PLANES) {
                    float4 h, l;
                    split_value(v[q].x, h.x, l.x); split_value(v[q].y, h.y, l.y); split_value(v[q].z, h.z, l.z); split_value(v[q].w, h.w, l.w);
                    *reinterpret_cast<float4 *>(hi + (r + q * kColsumRows) * pitch + col0) = h;
                    *reinterpret_cast<float4 *>(lo + (r + q * kColsumRows) * pitch + col0) = l;
                }
            }
        }
        for (; r < r1; r += kColsumRows) {
            float4 v = *reinterpret_cast<const float4 *>(g + r * cols + col0);
            a0 += v.x; a1 += v.y; a2 += v.z; a3 += v.w;
            if (PLANES) {
                float4 h, l;
                split_value(v.x, h.x, l.x); split_value(v.y, h.y, l.y); split_value(v.z, h.z, l.z); split_value(v.w, h.w, l.w);
                *reinterpret_cast<float4 *>(hi + r * pitch + col0) = h;
                *reinterpret_cast<float4 *>(lo + r * pitch + col0) = l;
            }
        }
    } else {
        for (int64_t r = r0 + w; r < r1; r += kColsumRows) {
            const float *row = g + r * cols;
            if (col0 < cols) a0 += row[col0];
            if (col0 + 1 < cols) a1 += row[col0 + 1];
            if (col0 + 2 < cols) a2 += row[col0 + 2];
            if (col0 + 3 < cols) a3 += row[col0 + 3];
        }
    }
    sm[w][lane * 4] = a0; sm[w][lane * 4 + 1] = a1; sm[w][lane * 4 + 2] = a2; sm[w][lane * 4 + 3] = a3;
    __syncthreads();
    if (threadIdx.x < 128) {
        double s = 0;
        for (int i = 0; i < kColsumRows; i++) s += sm[i][threadIdx.x];
        int64_t col = (int64_t)blockIdx.x * 128 + threadIdx.x;
        if (col < cols) partials[(int64_t)blockIdx.y * cols + col] = s;
    }
}
__global__ void colsum_final_kernel(const double *__restrict__ partials, int64_t splits, int64_t cols, float *out) {
    int64_t col = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (col >= cols) return;
    double s = 0;
    for (int64_t i = 0; i < splits; i++) s += partials[i * cols + col];
    out[col] = (float)s;
}

// Phase 2 for narrow matrices (few columns, many row splits): one warp per column, lanes stride over the
// splits and a fixed shuffle tree joins them, instead of one thread walking all the splits of a column
// (1024 sequential additions for the 10-wide head at batch 65536: 0.11 ms for 80 KB of partials).
__global__ void __launch_bounds__(256) colsum_final_narrow_kernel(const double *__restrict__ partials, int64_t splits, int64_t cols, float *out) {
    const int lane = threadIdx.x & 31;
    const int64_t col = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (col >= cols) return;
    double s = 0;
    for (int64_t i = lane; i < splits; i += 32) s += partials[i * cols + col];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) out[col] = (float)s;
}

inline int64_t colsum_splits(int64_t rows, int64_t cols) {
    int64_t strips = (cols + 127) / 128;
    int64_t want = (148 * 8 + strips - 1) / strips;            // about eight blocks per SM in total
    int64_t most = (rows + 63) / 64;                           // at least 64 rows per block
    int64_t s = want < most ? want : most;
    return s < 1 ? 1 : s;
}

// ---- index cross entropy with logits -----------------------------------------------------------
// Forward per row (CpuLossReferenceKernel.java:196-218,276-288): m = plain '>' maximum,
// s = sum exp(x - m), loss = (m + log s) - x[label].  The reference adds the exponentials in
// ascending binary32 order; here lanes add in binary64 and round once, which lies inside the
// reference's own rounding error of that sum.  Gradient (LossGradientRules.java:172-228):
// (exp(x - MAX) / SUM - onehot) * (seed / rows), MAX by Math.max, SUM exactly rounded.
template <typename L>
__device__ __forceinline__ int64_t load_label(const void *labels, int64_t r) { return (int64_t)((const L *)labels)[r]; }

// One row, any values (NaN, infinities, signed zeros), any width: re-reads the row from memory for
// each pass.  The careful route of the fast kernel and the body of the generic kernel.
__device__ __noinline__ void ce_row_careful(const float *__restrict__ row, int64_t cols, int64_t safe, float scale,
                                            float *loss_out, float *grad_row, int64_t *argmax_out, int lane) {
    float mplain = __int_as_float(0xff800000), mjava = __int_as_float(0xff800000);
    unsigned long long best = 0;
    for (int64_t c = lane; c < cols; c += 32) {
        float x = row[c];
        mplain = x > mplain ? x : mplain;
        mjava = java_max(mjava, x);
        unsigned long long cand = ((unsigned long long)order_key(x) << 32) | (0xffffffffu - (uint32_t)c);
        best = cand > best ? cand : best;
    }
    mplain = warp_max_plain(mplain);
    mjava = warp_max_java(mjava);
    if (argmax_out) { best = warp_best(best); if (lane == 0) *argmax_out = (int64_t)(0xffffffffu - (uint32_t)(best & 0xffffffffu)); }
    double acc = 0.0;
    for (int64_t c = lane; c < cols; c += 32) acc += (double)exp_accurate(__fsub_rn(row[c], mplain));
    float sum = (float)warp_sum(acc);
    if (lane == 0 && loss_out) *loss_out = __fsub_rn(__fadd_rn(mplain, (float)log((double)sum)), row[safe]);
    if (grad_row) {
        // the gradient's MAX aggregate follows Math.max: a NaN logit poisons the whole row
        if (mplain != mjava) sum = __int_as_float(0x7fc00000);
        for (int64_t c = lane; c < cols; c += 32) {
            float p = __fdiv_rn(exp_accurate(__fsub_rn(row[c], mplain)), sum);
            grad_row[c] = __fmul_rn(__fsub_rn(p, c == safe ? 1.0f : 0.0f), scale);
        }
    }
}

template <int CHUNKS, typename L, bool GRAD, bool ARGMAX>
__global__ void __launch_bounds__(kThreads, CHUNKS >= 8 ? 3 : 4) ce_rows_vec_kernel(const float *__restrict__ logits, const void *__restrict__ labels,
        const float *__restrict__ seed, int64_t rows, int cols, float *row_loss, float *grad, int64_t *argmax_out, int *error_word,
        int has_ignore, long long ignore, int scale_mode, const float *__restrict__ divisor) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int vec_cols = cols >> 2;
    // the cotangent each row's (p - onehot) is multiplied by: seed / rows (MEAN; under an ignore index
    // seed / rows that are left, counted into `divisor`), seed (SUM), seed[r] (NONE)
    const float uniform_scale = !GRAD ? 0.0f : scale_mode == 0 ? __fdiv_rn(seed ? seed[0] : 1.0f, divisor ? divisor[0] : (float)rows) : (seed ? seed[0] : 1.0f);
    for (int64_t r = warp; r < rows; r += warps) {
        const float scale = (GRAD && scale_mode == 2) ? seed[r] : uniform_scale;
        const float *row_s = logits + r * cols;
        const float4 *row = reinterpret_cast<const float4 *>(row_s);
        float4 v[CHUNKS];
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) v[j] = lane + 32 * j < vec_cols ? row[lane + 32 * j] : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        // the row this warp takes next, asked into L2 now (one 128-byte line per lane): its loads then
        // wait for L2 instead of HBM, which is what the six warps per scheduler could not hide
        if (r + warps < rows && lane * 32 < cols)
            asm volatile("prefetch.global.L2 [%0];" :: "l"(row_s + warps * cols + lane * 32));
        int64_t label = load_label<L>(labels, r);
        if (has_ignore && label == ignore) {
            // the ignore index is tested before the bounds and before the logits are read
            // (CpuLossReferenceKernel.java:261-265): zero loss, zero gradient
            if (lane == 0 && row_loss) row_loss[r] = 0.0f;
            if (GRAD) for (int c = lane; c < cols; c += 32) grad[r * cols + c] = 0.0f;
            if (ARGMAX) ce_row_careful(row_s, cols, 0, 0.0f, nullptr, nullptr, argmax_out + r, lane);
            continue;
        }
        if ((label < 0 || label >= cols) && lane == 0) atomicOr(error_word, ERR_LABEL_RANGE);
        const int safe = (int)(label < 0 ? 0 : (label >= cols ? cols - 1 : label));
        // maximum (fmaxf skips NaN like the reference's plain '>' scan) and a probe that turns NaN
        // for any NaN or infinity in the row: x * 0 accumulates on the FMA pipe
        float mplain = __int_as_float(0xff800000), probe = 0.0f;
        float m4[CHUNKS];                   // maximum of each 16-byte group, kept for the arg-max search
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            m4[j] = fmaxf(fmaxf(v[j].x, v[j].y), fmaxf(v[j].z, v[j].w));
            mplain = fmaxf(mplain, m4[j]);
            probe = fmaf(v[j].x, 0.0f, probe); probe = fmaf(v[j].y, 0.0f, probe);
            probe = fmaf(v[j].z, 0.0f, probe); probe = fmaf(v[j].w, 0.0f, probe);
        }
        mplain = warp_max_plain(mplain);
        const bool careful = __any_sync(0xffffffffu, probe != probe) || (ARGMAX && mplain == 0.0f);
        if (careful) {      // rare: non-finite logits, or a zero maximum whose sign decides the arg-max
            ce_row_careful(row_s, cols, safe, scale, row_loss ? row_loss + r : nullptr, GRAD ? grad + r * cols : nullptr,
                           ARGMAX ? argmax_out + r : nullptr, lane);
            continue;
        }
        if (ARGMAX) {       // finite row, non-zero maximum: the first column equal to it
            // only a group whose own maximum is the row maximum can hold it: one compare per group,
            // the four per-element compares only inside such a group
            uint32_t first = 0xffffffffu;
#pragma unroll
            for (int j = CHUNKS - 1; j >= 0; j--) {
                if (m4[j] == mplain) {
                    const uint32_t c4 = (uint32_t)(lane + 32 * j) * 4;
                    first = v[j].w == mplain ? c4 + 3 : first;
                    first = v[j].z == mplain ? c4 + 2 : first;
                    first = v[j].y == mplain ? c4 + 1 : first;
                    first = v[j].x == mplain ? c4 : first;
                }
            }
            first = warp_umin(first);
            if (lane == 0) argmax_out[r] = (int64_t)first;
        }
        double acc = 0.0;
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            // padding lanes hold -FLT_MAX: their exponential clamps to 1.18e-38, far below rounding
            float e0 = exp_shifted(__fsub_rn(v[j].x, mplain)), e1 = exp_shifted(__fsub_rn(v[j].y, mplain));
            float e2 = exp_shifted(__fsub_rn(v[j].z, mplain)), e3 = exp_shifted(__fsub_rn(v[j].w, mplain));
            v[j] = make_float4(e0, e1, e2, e3);
            if (lane + 32 * j < vec_cols) acc += (double)__fadd_rn(__fadd_rn(e0, e1), __fadd_rn(e2, e3));
        }
        const float sum = (float)warp_sum(acc);            // finite, at least 1: the maximum contributes exp(0)
        const int owner = (safe >> 2) & 31;
        const float target_logit = row_s[safe];            // a cache hit; avoids selecting it out of the registers
        if (lane == 0 && row_loss) row_loss[r] = __fsub_rn(__fadd_rn(mplain, (float)log((double)sum)), target_logit);
        if (GRAD) {
            float4 *out = reinterpret_cast<float4 *>(grad + r * cols);
            // p = e / sum as one reciprocal per row plus a remainder-corrected product per element;
            // (p - onehot) * scale equals p * scale everywhere but at the label, which its owner fixes up
            const float rcp = __frcp_rn(sum);
#pragma unroll
            for (int j = 0; j < CHUNKS; j++) {
                float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float p = __fmul_rn(e[q], rcp);
                    p = fmaf(fmaf(-p, sum, e[q]), rcp, p);
                    e[q] = __fmul_rn(p, scale);
                }
                if (lane + 32 * j < vec_cols) out[lane + 32 * j] = make_float4(e[0], e[1], e[2], e[3]);
            }
            if (lane == owner) {
                const float te = exp_shifted(__fsub_rn(target_logit, mplain));
                float p = __fmul_rn(te, rcp);
                p = fmaf(fmaf(-p, sum, te), rcp, p);
                grad[r * cols + safe] = __fmul_rn(__fsub_rn(p, 1.0f), scale);     // same thread as the float4 store above: ordered
            }
        }
    }
}

// Any column count: one warp per row through the careful routine; used for narrow rows (the
// 10-class head) and rows that are not 16-byte aligned.
template <typename L>
__global__ void ce_rows_generic_kernel(const float *__restrict__ logits, const void *__restrict__ labels, const float *__restrict__ seed,
        int64_t rows, int64_t cols, float *row_loss, float *grad, int64_t *argmax_out, int *error_word,
        int has_ignore, long long ignore, int scale_mode, const float *__restrict__ divisor) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const float uniform_scale = !grad ? 0.0f : scale_mode == 0 ? __fdiv_rn(seed ? seed[0] : 1.0f, divisor ? divisor[0] : (float)rows) : (seed ? seed[0] : 1.0f);
    for (int64_t r = warp; r < rows; r += warps) {
        const float scale = (grad && scale_mode == 2) ? seed[r] : uniform_scale;
        int64_t label = load_label<L>(labels, r);
        if (has_ignore && label == ignore) {
            if (lane == 0 && row_loss) row_loss[r] = 0.0f;
            if (grad) for (int64_t c = lane; c < cols; c += 32) grad[r * cols + c] = 0.0f;
            if (argmax_out) ce_row_careful(logits + r * cols, cols, 0, 0.0f, nullptr, nullptr, argmax_out + r, lane);
            continue;
        }
        if ((label < 0 || label >= cols) && lane == 0) atomicOr(error_word, ERR_LABEL_RANGE);
        int64_t safe = label < 0 ? 0 : (label >= cols ? cols - 1 : label);
        ce_row_careful(logits + r * cols, cols, safe, scale, row_loss ? row_loss + r : nullptr, grad ? grad + r * cols : nullptr,
                       argmax_out ? argmax_out + r : nullptr, lane);
    }
}

// Mean of the per-row losses: the reference adds them in ascending binary32 order and divides by
// the count; one block adds them in binary64 in a fixed order and rounds once.
__global__ void mean_kernel(const float *__restrict__ values, int64_t count, float *out, int divide) {
    __shared__ double partial[32];
    double acc = 0.0;
    if ((count & 3) == 0 && ((uintptr_t)values & 15) == 0) {
        // 16-byte loads, four of them in flight per thread: one block reading scalars one by one is
        // bound by load latency (12 us for 65536 row losses)
        const float4 *v4 = reinterpret_cast<const float4 *>(values);
        const int64_t n4 = count >> 2;
        int64_t i = threadIdx.x;
        for (; i + 3 * (int64_t)blockDim.x < n4; i += 4 * (int64_t)blockDim.x) {
            float4 q[4];
#pragma unroll
            for (int u = 0; u < 4; u++) q[u] = v4[i + u * (int64_t)blockDim.x];
#pragma unroll
            for (int u = 0; u < 4; u++) acc += ((double)q[u].x + (double)q[u].y) + ((double)q[u].z + (double)q[u].w);
        }
        for (; i < n4; i += blockDim.x) { float4 q = v4[i]; acc += ((double)q.x + (double)q.y) + ((double)q.z + (double)q.w); }
    } else {
        for (int64_t i = threadIdx.x; i < count; i += blockDim.x) acc += (double)values[i];
    }
    acc = warp_sum(acc);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        double v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.0;
        v = warp_sum(v);
        if (threadIdx.x == 0) out[0] = divide ? __fdiv_rn((float)v, (float)count) : (float)v;
    }
}

// Reduction of the row losses under an ignore index (CpuLossReferenceKernel.java:208-218): ignored
// rows add nothing and are not counted; MEAN divides by the number of rows that are left (0 / 0 is
// NaN when every row is ignored, as there).
// Number of rows whose label is not the ignore index, as the binary32 value the rule's exactly
// rounded SUM over its zeros and ones gives.
template <typename L>
__global__ void count_active_kernel(const void *__restrict__ labels, long long ignore, int64_t count, float *out) {
    __shared__ long long partial[32];
    long long active = 0;
    for (int64_t i = threadIdx.x; i < count; i += blockDim.x) active += load_label<L>(labels, i) != ignore;
    for (int o = 16; o > 0; o >>= 1) active += __shfl_xor_sync(0xffffffffu, active, o);
    if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = active;
    __syncthreads();
    if (threadIdx.x < 32) {
        long long n = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0;
        for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
        if (threadIdx.x == 0) out[0] = (float)n;
    }
}

template <typename L>
__global__ void mean_active_kernel(const float *__restrict__ values, const void *__restrict__ labels, long long ignore, int64_t count,
                                   float *out, int divide) {
    __shared__ double partial[32];
    __shared__ long long active_partial[32];
    double acc = 0.0;
    long long active = 0;
    for (int64_t i = threadIdx.x; i < count; i += blockDim.x)
        if (load_label<L>(labels, i) != ignore) { acc += (double)values[i]; active++; }
    acc = warp_sum(acc);
    for (int o = 16; o > 0; o >>= 1) active += __shfl_xor_sync(0xffffffffu, active, o);
    if ((threadIdx.x & 31) == 0) { partial[threadIdx.x >> 5] = acc; active_partial[threadIdx.x >> 5] = active; }
    __syncthreads();
    if (threadIdx.x < 32) {
        double v = threadIdx.x < (blockDim.x >> 5) ? partial[threadIdx.x] : 0.0;
        long long n = threadIdx.x < (blockDim.x >> 5) ? active_partial[threadIdx.x] : 0;
        v = warp_sum(v);
        for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
        if (threadIdx.x == 0) out[0] = divide ? __fdiv_rn((float)v, (float)n) : (float)v;
    }
}

// ---- dense-target categorical cross entropy with logits, forward --------------------------------
// Per row (CpuLossReferenceKernel.java:129-143,251-259,276-288): lse = m + (float)log(sum exp(x - m))
// with the plain '>' maximum, then the sum over the classes whose target weight is not zero of
// weight * (lse - x), each term rounded to binary32.  The reference adds the exponentials and the
// terms in ascending binary32 order; here lanes add in binary64 and round once, which lies inside
// the reference's own rounding error of those sums.  One warp per row, the row read twice (the
// second pass hits L1 / L2).
// One row, any values and any width.
__device__ __forceinline__ float dense_ce_row_careful(const float *__restrict__ row, const float *__restrict__ weight, int64_t cols, int lane) {
    float mplain = __int_as_float(0xff800000);
    for (int64_t c = lane; c < cols; c += 32) { float x = row[c]; mplain = x > mplain ? x : mplain; }
    mplain = warp_max_plain(mplain);
    double acc = 0.0;
    for (int64_t c = lane; c < cols; c += 32) acc += (double)exp_accurate(__fsub_rn(row[c], mplain));
    const float sum = (float)warp_sum(acc);
    const float lse = __fadd_rn(mplain, (float)log((double)sum));
    double loss = 0.0;
    for (int64_t c = lane; c < cols; c += 32) {
        const float w = weight[c];
        if (w != 0.0f) loss += (double)__fmul_rn(w, __fsub_rn(lse, row[c]));
    }
    return (float)warp_sum(loss);
}

__global__ void dense_ce_rows_kernel(const float *__restrict__ logits, const float *__restrict__ target, int64_t rows, int64_t cols,
                                     float *row_loss) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += warps) {
        const float loss = dense_ce_row_careful(logits + r * cols, target + r * cols, cols, lane);
        if (lane == 0) row_loss[r] = loss;
    }
}

// Rows of 128 to 1024 columns, 16-byte aligned: the logits are read once into registers (one warp
// per row), finite rows take the exponential once per element (exp_shifted), and the target weights
// stream past the cached logits; rows with an infinity or NaN among the logits go to the careful
// routine.  The next row's logits and weights are asked into L2 meanwhile.
template <int CHUNKS>
__global__ void __launch_bounds__(kThreads, CHUNKS >= 8 ? 2 : 4) dense_ce_rows_vec_kernel(const float *__restrict__ logits,
        const float *__restrict__ target, int64_t rows, int cols, float *row_loss) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int vec_cols = cols >> 2;
    for (int64_t r = warp; r < rows; r += warps) {
        const float *row_s = logits + r * cols;
        const float4 *row = reinterpret_cast<const float4 *>(row_s);
        const float4 *weight = reinterpret_cast<const float4 *>(target + r * cols);
        float4 v[CHUNKS];
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) v[j] = lane + 32 * j < vec_cols ? row[lane + 32 * j] : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
        // the weights are asked for together with the logits, so that their latency passes under the
        // exponentials instead of after them (asked for only when needed, the pass ran at 3.5 TB/s)
        float4 wv[CHUNKS];
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) wv[j] = lane + 32 * j < vec_cols ? weight[lane + 32 * j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (r + warps < rows && lane * 32 < cols) {
            asm volatile("prefetch.global.L2 [%0];" :: "l"(row_s + warps * cols + lane * 32));
            asm volatile("prefetch.global.L2 [%0];" :: "l"(target + (r + warps) * cols + lane * 32));
        }
        float mplain = __int_as_float(0xff800000), probe = 0.0f;
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            mplain = fmaxf(fmaxf(mplain, fmaxf(v[j].x, v[j].y)), fmaxf(v[j].z, v[j].w));
            probe = fmaf(v[j].x, 0.0f, probe); probe = fmaf(v[j].y, 0.0f, probe);
            probe = fmaf(v[j].z, 0.0f, probe); probe = fmaf(v[j].w, 0.0f, probe);
        }
        mplain = warp_max_plain(mplain);
        if (__any_sync(0xffffffffu, probe != probe)) {      // rare: an infinity or NaN among the logits
            const float loss = dense_ce_row_careful(row_s, target + r * cols, cols, lane);
            if (lane == 0) row_loss[r] = loss;
            continue;
        }
        double acc = 0.0;
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            const float e0 = exp_shifted(__fsub_rn(v[j].x, mplain)), e1 = exp_shifted(__fsub_rn(v[j].y, mplain));
            const float e2 = exp_shifted(__fsub_rn(v[j].z, mplain)), e3 = exp_shifted(__fsub_rn(v[j].w, mplain));
            if (lane + 32 * j < vec_cols) acc += (double)__fadd_rn(__fadd_rn(e0, e1), __fadd_rn(e2, e3));
        }
        const float sum = (float)warp_sum(acc);
        const float lse = __fadd_rn(mplain, (float)log((double)sum));
        double loss = 0.0;
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            {
                const float4 w = wv[j];                 // zero past the row's end
                // a zero weight contributes nothing, whatever lse - x is (the reference skips it)
                const float t0 = w.x != 0.0f ? __fmul_rn(w.x, __fsub_rn(lse, v[j].x)) : 0.0f, t1 = w.y != 0.0f ? __fmul_rn(w.y, __fsub_rn(lse, v[j].y)) : 0.0f;
                const float t2 = w.z != 0.0f ? __fmul_rn(w.z, __fsub_rn(lse, v[j].z)) : 0.0f, t3 = w.w != 0.0f ? __fmul_rn(w.w, __fsub_rn(lse, v[j].w)) : 0.0f;
                // four terms are added in binary32 first: one binary64 addition per group keeps the FP64 pipe
                // out of the way (the reference adds all terms in binary32)
                loss += (double)__fadd_rn(__fadd_rn(t0, t1), __fadd_rn(t2, t3));
            }
        }
        loss = warp_sum(loss);
        if (lane == 0) row_loss[r] = (float)loss;
    }
}

// ---- dense-target categorical cross entropy, gradient with respect to the logits -----------------
// The node list of LossGradientRules.denseCategorical (:131-145) in one pass per row:
// (p * mass - target) * scale with p = exp(x - MAX) / SUM(exp(x - MAX)) (aggregate MAX by Math.max, so a
// NaN logit poisons its row), mass = SUM(target) exactly rounded, every product and difference a
// separate binary32 rounding; a row whose targets are all zero gives zeros.  scale as in the index form:
// seed / rows, seed, or seed[row].
__device__ __forceinline__ void dense_ce_grad_row_careful(const float *__restrict__ row, const float *__restrict__ weight, int64_t cols,
                                                          float scale, float *grad_row, int lane) {
    double mass_acc = 0.0;
    int any = 0;
    float mjava = __int_as_float(0xff800000);
    for (int64_t c = lane; c < cols; c += 32) {
        const float w = weight[c];
        mass_acc += (double)w; any |= w != 0.0f;             // NaN != 0: a NaN weight counts as a member
        mjava = java_max(mjava, row[c]);
    }
    any = __any_sync(0xffffffffu, any);
    if (!any) { for (int64_t c = lane; c < cols; c += 32) grad_row[c] = 0.0f; return; }
    const float mass = (float)warp_sum(mass_acc);
    mjava = warp_max_java(mjava);
    double acc = 0.0;
    for (int64_t c = lane; c < cols; c += 32) acc += (double)exp_accurate(__fsub_rn(row[c], mjava));
    const float sum = (float)warp_sum(acc);
    for (int64_t c = lane; c < cols; c += 32) {
        const float p = __fdiv_rn(exp_accurate(__fsub_rn(row[c], mjava)), sum);
        grad_row[c] = __fmul_rn(__fsub_rn(__fmul_rn(p, mass), weight[c]), scale);
    }
}

__global__ void dense_ce_grad_rows_kernel(const float *__restrict__ logits, const float *__restrict__ target, const float *__restrict__ seed,
                                          int64_t rows, int64_t cols, float *grad, int scale_mode) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const float uniform_scale = scale_mode == 0 ? __fdiv_rn(seed ? seed[0] : 1.0f, (float)rows) : (seed ? seed[0] : 1.0f);
    for (int64_t r = warp; r < rows; r += warps)
        dense_ce_grad_row_careful(logits + r * cols, target + r * cols, cols, scale_mode == 2 ? seed[r] : uniform_scale, grad + r * cols, lane);
}

// Rows of 128 to 1024 columns, 16-byte aligned: logits and weights are read once into registers (asked
// for together), finite rows take one exponential per element and the quotient as a reciprocal per row
// with a remainder-corrected product per element.
template <int CHUNKS>
__global__ void __launch_bounds__(kThreads, CHUNKS >= 8 ? 2 : 4) dense_ce_grad_rows_vec_kernel(const float *__restrict__ logits,
        const float *__restrict__ target, const float *__restrict__ seed, int64_t rows, int cols, float *grad, int scale_mode) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int vec_cols = cols >> 2;
    const float uniform_scale = scale_mode == 0 ? __fdiv_rn(seed ? seed[0] : 1.0f, (float)rows) : (seed ? seed[0] : 1.0f);
    for (int64_t r = warp; r < rows; r += warps) {
        const float scale = scale_mode == 2 ? seed[r] : uniform_scale;
        const float *row_s = logits + r * cols;
        const float4 *row = reinterpret_cast<const float4 *>(row_s);
        const float4 *weight = reinterpret_cast<const float4 *>(target + r * cols);
        float4 v[CHUNKS], wv[CHUNKS];
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) v[j] = lane + 32 * j < vec_cols ? row[lane + 32 * j] : make_float4(-FLT_MAX, -FLT_MAX, -FLT_MAX, -FLT_MAX);
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) wv[j] = lane + 32 * j < vec_cols ? weight[lane + 32 * j] : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (r + warps < rows && lane * 32 < cols) {
            asm volatile("prefetch.global.L2 [%0];" :: "l"(row_s + warps * cols + lane * 32));
            asm volatile("prefetch.global.L2 [%0];" :: "l"(target + (r + warps) * cols + lane * 32));
        }
        float maximum = __int_as_float(0xff800000), probe = 0.0f;
        double mass_acc = 0.0;
        int any = 0;
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            maximum = fmaxf(fmaxf(maximum, fmaxf(v[j].x, v[j].y)), fmaxf(v[j].z, v[j].w));
            probe = fmaf(v[j].x, 0.0f, probe); probe = fmaf(v[j].y, 0.0f, probe);
            probe = fmaf(v[j].z, 0.0f, probe); probe = fmaf(v[j].w, 0.0f, probe);
            mass_acc += ((double)wv[j].x + (double)wv[j].y) + ((double)wv[j].z + (double)wv[j].w);
            any |= (wv[j].x != 0.0f) | (wv[j].y != 0.0f) | (wv[j].z != 0.0f) | (wv[j].w != 0.0f);
        }
        maximum = warp_max_plain(maximum);
        if (__any_sync(0xffffffffu, probe != probe)) {      // rare: an infinity or NaN among the logits
            dense_ce_grad_row_careful(row_s, target + r * cols, cols, scale, grad + r * cols, lane);
            continue;
        }
        float4 *out = reinterpret_cast<float4 *>(grad + r * cols);
        if (!__any_sync(0xffffffffu, any)) {                // no target mass in this row: no gradient
#pragma unroll
            for (int j = 0; j < CHUNKS; j++) if (lane + 32 * j < vec_cols) out[lane + 32 * j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            continue;
        }
        const float mass = (float)warp_sum(mass_acc);
        double acc = 0.0;
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            const float e0 = exp_shifted(__fsub_rn(v[j].x, maximum)), e1 = exp_shifted(__fsub_rn(v[j].y, maximum));
            const float e2 = exp_shifted(__fsub_rn(v[j].z, maximum)), e3 = exp_shifted(__fsub_rn(v[j].w, maximum));
            v[j] = make_float4(e0, e1, e2, e3);
            if (lane + 32 * j < vec_cols) acc += (double)__fadd_rn(__fadd_rn(e0, e1), __fadd_rn(e2, e3));
        }
        const float sum = (float)warp_sum(acc);
        const float rcp = __frcp_rn(sum);
#pragma unroll
        for (int j = 0; j < CHUNKS; j++) {
            float e[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
            const float t[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                float p = __fmul_rn(e[q], rcp);
                p = fmaf(fmaf(-p, sum, e[q]), rcp, p);
                e[q] = __fmul_rn(__fsub_rn(__fmul_rn(p, mass), t[q]), scale);
            }
            if (lane + 32 * j < vec_cols) out[lane + 32 * j] = make_float4(e[0], e[1], e[2], e[3]);
        }
    }
}

// ---- optimizers --------------------------------------------------------------------------------
constexpr int kMaxSlots = 40;       // the table travels as a kernel argument: 40 slots keep it under 4 KB
struct SlotTable { TensorSlot slot[kMaxSlots]; int64_t first_block[kMaxSlots + 1]; int count; };
constexpr int kOptElemsPerBlock = kThreads * 8;

__device__ __forceinline__ bool finite(float x) { return (__float_as_uint(x) & 0x7f800000u) != 0x7f800000u; }

// True when an earlier launch on this context has already reported a failure: the step this kernel
// belongs to must then leave no trace.  The first thread records the step as not taken.
__device__ __forceinline__ bool step_is_void(const int *error_word, int sequence, int *failed_sequence) {
    if (*reinterpret_cast<const volatile int *>(error_word) == 0) return false;
    if (blockIdx.x == 0 && threadIdx.x == 0) atomicMin(failed_sequence, sequence);
    return true;
}

// SGD, TrainingParameter.java:622-672: every product and sum is a separate binary32 rounding.  Reads
// p, m, acc, g; writes the candidates p_out, m_out.
__global__ void __launch_bounds__(kThreads) sgd_kernel(SlotTable table, SgdArgs a, int *error_word) {
    if (step_is_void(error_word, a.sequence, a.failed_sequence)) return;
    int t = 0;
    while (t + 1 < table.count && (int64_t)blockIdx.x >= table.first_block[t + 1]) t++;
    const TensorSlot s = table.slot[t];
    int64_t base = ((int64_t)blockIdx.x - table.first_block[t]) * kOptElemsPerBlock;
    bool bad = false;
    for (int64_t i = base + threadIdx.x; i < base + kOptElemsPerBlock && i < s.count; i += kThreads) {
        float p = s.p[i];
        float g = s.g[i];
        if (a.gradient_mode == 2) { g = __fadd_rn(s.acc[i], g); bad |= !finite(g); }
        float decay_term = __fmul_rn(a.weight_decay, p);
        float adjusted = __fadd_rn(g, decay_term);
        float update = adjusted;
        if (a.momentum != 0.0f) {
            float buf;
            if (a.first_step) buf = adjusted;
            else buf = __fadd_rn(__fmul_rn(a.momentum, s.m[i]), __fmul_rn(__fsub_rn(1.0f, a.dampening), adjusted));
            s.m_out[i] = buf;
            update = a.nesterov ? __fadd_rn(adjusted, __fmul_rn(a.momentum, buf)) : buf;
            bad |= !finite(buf);
        } else if (a.zero_buffer) s.m_out[i] = 0.0f;
        float scaled = __fmul_rn(a.lr, update);
        float candidate = __fsub_rn(p, scaled);
        bad |= !finite(p) || !finite(decay_term) || !finite(adjusted) || !finite(update) || !finite(scaled) || !finite(candidate);
        s.p_out[i] = candidate;
    }
    if (bad) { atomicOr(error_word, ERR_NON_FINITE); atomicMin(a.failed_sequence, a.sequence); }
}

// Adam / AdamW, TrainingParameter.java:433-525: m = b1*m + (1-b1)*g; v = b2*v + (1-b2)*(g*g);
// update = (lr * (m / c1)) / (sqrt(v / c2) + eps), the product formed before the division.  Reads
// p, m, v, acc, g; writes the candidates p_out, m_out, v_out (28 bytes per parameter either way).
// One element; returns true when any intermediate is non-finite.
__device__ __forceinline__ bool adam_element(const AdamArgs &a, float one_minus_b1, float one_minus_b2, float p, float g, float pending,
                                             float m0, float v0, float &p_new, float &m_new, float &v_new) {
    bool bad = false;
    float basev;
    if (a.gradient_mode == 2) { g = __fadd_rn(pending, g); bad |= !finite(g); }
    if (a.decoupled) basev = __fmul_rn(p, a.decay_factor);
    else { g = __fadd_rn(g, __fmul_rn(a.decay, p)); basev = p; }
    const float m = __fadd_rn(__fmul_rn(a.b1, m0), __fmul_rn(one_minus_b1, g));
    const float sq = __fmul_rn(g, g);
    const float v = __fadd_rn(__fmul_rn(a.b2, v0), __fmul_rn(one_minus_b2, sq));
    const float mh = __fdiv_rn(m, a.correction1), vh = __fdiv_rn(v, a.correction2);
    const float den = __fadd_rn(__fsqrt_rn(vh), a.eps);
    const float num = __fmul_rn(a.lr, mh);
    const float update = __fdiv_rn(num, den);
    const float candidate = __fsub_rn(basev, update);
    bad |= !finite(p) || !finite(g) || !finite(m) || !finite(sq) || !finite(v) || !finite(mh) || !finite(vh)
           || !finite(den) || !(den > 0.0f) || !finite(num) || !finite(update) || !finite(candidate);
    p_new = candidate; m_new = m; v_new = v;
    return bad;
}

__global__ void __launch_bounds__(kThreads) adam_kernel(SlotTable table, AdamArgs a, int *error_word) {
    if (step_is_void(error_word, a.sequence, a.failed_sequence)) return;
    int t = 0;
    while (t + 1 < table.count && (int64_t)blockIdx.x >= table.first_block[t + 1]) t++;
    const TensorSlot s = table.slot[t];
    const int64_t base = ((int64_t)blockIdx.x - table.first_block[t]) * kOptElemsPerBlock;
    const int64_t end = base + kOptElemsPerBlock < s.count ? base + kOptElemsPerBlock : s.count;
    const float one_minus_b1 = __fsub_rn(1.0f, a.b1), one_minus_b2 = __fsub_rn(1.0f, a.b2);
    const bool with_pending = a.gradient_mode == 2;
    bool bad = false;
    // 16-byte loads and stores (the block's first element is a multiple of 2048, so alignment is that of
    // the arrays themselves); whatever is left at the end of the tensor goes element by element
    const bool vec = ((((uintptr_t)s.p | (uintptr_t)s.g | (uintptr_t)s.m | (uintptr_t)s.v | (uintptr_t)s.p_out | (uintptr_t)s.m_out
                        | (uintptr_t)s.v_out | (with_pending ? (uintptr_t)s.acc : 0)) & 15) == 0);
    int64_t scalar_from = base;
    if (vec) {
        const int64_t quads = (end - base) >> 2;
        for (int64_t q = threadIdx.x; q < quads; q += kThreads) {
            const int64_t i = base + (q << 2);
            const float4 p = *reinterpret_cast<const float4 *>(s.p + i), g = *reinterpret_cast<const float4 *>(s.g + i);
            const float4 m = *reinterpret_cast<const float4 *>(s.m + i), v = *reinterpret_cast<const float4 *>(s.v + i);
            float4 pending = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (with_pending) pending = *reinterpret_cast<const float4 *>(s.acc + i);
            float4 pn, mn, vn;
            bad |= adam_element(a, one_minus_b1, one_minus_b2, p.x, g.x, pending.x, m.x, v.x, pn.x, mn.x, vn.x);
            bad |= adam_element(a, one_minus_b1, one_minus_b2, p.y, g.y, pending.y, m.y, v.y, pn.y, mn.y, vn.y);
            bad |= adam_element(a, one_minus_b1, one_minus_b2, p.z, g.z, pending.z, m.z, v.z, pn.z, mn.z, vn.z);
            bad |= adam_element(a, one_minus_b1, one_minus_b2, p.w, g.w, pending.w, m.w, v.w, pn.w, mn.w, vn.w);
            *reinterpret_cast<float4 *>(s.p_out + i) = pn;
            *reinterpret_cast<float4 *>(s.m_out + i) = mn;
            *reinterpret_cast<float4 *>(s.v_out + i) = vn;
        }
        scalar_from = base + (quads << 2);
    }
    for (int64_t i = scalar_from + threadIdx.x; i < end; i += kThreads) {
        float pn, mn, vn;
        bad |= adam_element(a, one_minus_b1, one_minus_b2, s.p[i], s.g[i], with_pending ? s.acc[i] : 0.0f, s.m[i], s.v[i], pn, mn, vn);
        s.p_out[i] = pn; s.m_out[i] = mn; s.v_out[i] = vn;
    }
    if (bad) { atomicOr(error_word, ERR_NON_FINITE); atomicMin(a.failed_sequence, a.sequence); }
}

// Zeroes the pending sums once the step that consumed (or dropped) them has gone through.
struct NoArgs {};
__global__ void __launch_bounds__(kThreads) clear_pending_kernel(SlotTable table, NoArgs, int *error_word) {
    if (*reinterpret_cast<const volatile int *>(error_word) != 0) return;
    int t = 0;
    while (t + 1 < table.count && (int64_t)blockIdx.x >= table.first_block[t + 1]) t++;
    const TensorSlot s = table.slot[t];
    int64_t base = ((int64_t)blockIdx.x - table.first_block[t]) * kOptElemsPerBlock;
    for (int64_t i = base + threadIdx.x; i < base + kOptElemsPerBlock && i < s.count; i += kThreads) s.acc[i] = 0.0f;
}

// GradientMode.ACCUMULATE (TrainingParameter.java:373-390): the pending sum takes one binary32 addition
// per run.  COMMIT false: only looks for a non-finite sum; COMMIT true: adds, unless anything has failed.
struct AccumulateArgs { int sequence; int *failed_sequence; };
template <bool COMMIT>
__global__ void __launch_bounds__(kThreads) accumulate_kernel(SlotTable table, AccumulateArgs a, int *error_word) {
    if (COMMIT) { if (*reinterpret_cast<const volatile int *>(error_word) != 0) return; }
    else if (step_is_void(error_word, a.sequence, a.failed_sequence)) return;
    int t = 0;
    while (t + 1 < table.count && (int64_t)blockIdx.x >= table.first_block[t + 1]) t++;
    const TensorSlot s = table.slot[t];
    int64_t base = ((int64_t)blockIdx.x - table.first_block[t]) * kOptElemsPerBlock;
    bool bad = false;
    for (int64_t i = base + threadIdx.x; i < base + kOptElemsPerBlock && i < s.count; i += kThreads) {
        float sum = __fadd_rn(s.acc[i], s.g[i]);
        if (COMMIT) s.acc[i] = sum; else bad |= !finite(sum);
    }
    if (bad) { atomicOr(error_word, ERR_NON_FINITE); atomicMin(a.failed_sequence, a.sequence); }
}

template <typename K, typename A>
cudaError_t launch_slots(cudaStream_t s, K kernel, const TensorSlot *slots, int slot_count, const A &args, int *error_word) {
    for (int first = 0; first < slot_count; first += kMaxSlots) {
        SlotTable table;
        table.count = slot_count - first < kMaxSlots ? slot_count - first : kMaxSlots;
        int64_t blocks = 0;
        for (int i = 0; i < table.count; i++) {
            table.slot[i] = slots[first + i];
            table.first_block[i] = blocks;
            blocks += (slots[first + i].count + kOptElemsPerBlock - 1) / kOptElemsPerBlock;
        }
        table.first_block[table.count] = blocks;
        if (blocks == 0) continue;
        kernel<<<(unsigned)blocks, kThreads, 0, s>>>(table, args, error_word);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

// ---- 16-bit storage: element-wise nodes and the row arg-max ---------------------------------------
// Operands widened to FLOAT32, the operation there, one narrowing (CpuScalarReferenceKernel.java:93-115,
// arithmetic :975-985).
template <int KIND>
__global__ void binary_low_kernel(int op, const uint16_t *__restrict__ a, const uint16_t *__restrict__ b, uint16_t *out, Index4 ix, int64_t total) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t oa, ob, oc;
        unravel(i, ix, oa, ob, oc);
        const float x = low_decode<KIND>(a[oa]), y = low_decode<KIND>(b[ob]);
        float r;
        switch ((Op)op) {
            case Op::ADD: r = __fadd_rn(x, y); break;
            case Op::SUB: r = __fsub_rn(x, y); break;
            case Op::MUL: r = __fmul_rn(x, y); break;
            default: r = __fdiv_rn(x, y); break;
        }
        out[i] = low_encode<KIND>(r);
    }
}

template <int KIND>
__global__ void unary_low_kernel(int op, const uint16_t *__restrict__ a, uint16_t *out, int64_t total) {
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
        out[i] = low_encode<KIND>(low_activation_value(op, low_decode<KIND>(a[i])));
}

template <int KIND>
__global__ void __launch_bounds__(kThreads) argmax_low_kernel(const uint16_t *__restrict__ x, int64_t *out, int64_t rows, int64_t cols) {
    int lane = threadIdx.x & 31;
    int64_t warp = (blockIdx.x * (int64_t)blockDim.x + threadIdx.x) >> 5, warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t r = warp; r < rows; r += warps) {
        const uint16_t *row = x + r * cols;
        unsigned long long best = 0;        // larger key wins; among equal keys the smaller index (FIRST_INDEX ties)
        for (int64_t c = lane; c < cols; c += 32) {
            unsigned long long cand = ((unsigned long long)order_key(low_decode<KIND>(row[c])) << 32) | (0xffffffffu - (uint32_t)c);
            best = cand > best ? cand : best;
        }
        best = warp_best(best);
        if (lane == 0) out[r] = (int64_t)(0xffffffffu - (uint32_t)(best & 0xffffffffu));
    }
}

}  // namespace

cudaError_t binary(cudaStream_t s, Op op, const float *a, const float *b, void *out, const Index4 &ix, int64_t total) {
    if (total == 0) return cudaSuccess;
    binary_kernel<<<grid_for(total, kThreads), kThreads, 0, s>>>((int)op, a, b, out, ix, total);
    return cudaGetLastError();
}

cudaError_t binary_int(cudaStream_t s, Op op, DType dtype, const void *a, const void *b, void *out, const Index4 &ix, int64_t total) {
    if (total == 0) return cudaSuccess;
    if (op != Op::SUB && op != Op::EQ) return cudaErrorInvalidValue;
    if (dtype == DType::I32) binary_int_kernel<int32_t><<<grid_for(total, kThreads), kThreads, 0, s>>>((int)op, (const int32_t *)a, (const int32_t *)b, out, ix, total);
    else if (dtype == DType::I64) binary_int_kernel<int64_t><<<grid_for(total, kThreads), kThreads, 0, s>>>((int)op, (const int64_t *)a, (const int64_t *)b, out, ix, total);
    else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t where(cudaStream_t s, const uint8_t *cond, const float *a, const float *b, float *out, const Index4 &ix, int64_t total) {
    if (total == 0) return cudaSuccess;
    where_kernel<<<grid_for(total, kThreads), kThreads, 0, s>>>(cond, a, b, out, ix, total);
    return cudaGetLastError();
}

cudaError_t scalar_op(cudaStream_t s, Op op, DType dtype, const void *a, void *out, uint64_t scalar_bits, int64_t total) {
    if (total == 0) return cudaSuccess;
    int grid = grid_for(total, kThreads);
    if (dtype == DType::F32) {
        double d; memcpy(&d, &scalar_bits, 8);
        scalar_f32_kernel<<<grid, kThreads, 0, s>>>((int)op, (const float *)a, (float *)out, (float)d, total);
    } else if (dtype == DType::I32) {
        scalar_kernel<int32_t><<<grid, kThreads, 0, s>>>((int)op, (const int32_t *)a, (int32_t *)out, (int32_t)(int64_t)scalar_bits, total);
    } else if (dtype == DType::I64) {
        scalar_kernel<int64_t><<<grid, kThreads, 0, s>>>((int)op, (const int64_t *)a, (int64_t *)out, (int64_t)scalar_bits, total);
    } else return cudaErrorInvalidValue;
    return cudaGetLastError();
}

cudaError_t unary(cudaStream_t s, Op op, const float *a, void *out, int64_t total) {
    if (total == 0) return cudaSuccess;
    unary_kernel<<<grid_for(total, kThreads), kThreads, 0, s>>>((int)op, a, out, total);
    return cudaGetLastError();
}

cudaError_t one_hot(cudaStream_t s, DType index_type, const void *indices, uint8_t *out, int64_t count, int64_t depth) {
    if (count * depth == 0) return cudaSuccess;
    int grid = grid_for(count * depth, kThreads);
    if (index_type == DType::I32) one_hot_kernel<int32_t><<<grid, kThreads, 0, s>>>((const int32_t *)indices, out, count, depth);
    else one_hot_kernel<int64_t><<<grid, kThreads, 0, s>>>((const int64_t *)indices, out, count, depth);
    return cudaGetLastError();
}

cudaError_t copy_strided(cudaStream_t s, int element_bytes, const void *src, void *dst, const Index4 &ix, int64_t total) {
    if (total == 0) return cudaSuccess;
    int grid = grid_for(total, kThreads);
    if (element_bytes == 4) copy_kernel<uint32_t><<<grid, kThreads, 0, s>>>((const uint32_t *)src, (uint32_t *)dst, ix, total);
    else if (element_bytes == 8) copy_kernel<uint64_t><<<grid, kThreads, 0, s>>>((const uint64_t *)src, (uint64_t *)dst, ix, total);
    else if (element_bytes == 2) copy_kernel<uint16_t><<<grid, kThreads, 0, s>>>((const uint16_t *)src, (uint16_t *)dst, ix, total);
    else copy_kernel<uint8_t><<<grid, kThreads, 0, s>>>((const uint8_t *)src, (uint8_t *)dst, ix, total);
    return cudaGetLastError();
}

cudaError_t binary_low(cudaStream_t s, int kind, Op op, const void *a, const void *b, void *out, const Index4 &ix, int64_t total) {
    if (total == 0) return cudaSuccess;
    if ((kind != 1 && kind != 2) || (op != Op::ADD && op != Op::SUB && op != Op::MUL && op != Op::DIV)) return cudaErrorInvalidValue;
    const int grid = grid_for(total, kThreads);
    if (kind == 1) binary_low_kernel<1><<<grid, kThreads, 0, s>>>((int)op, (const uint16_t *)a, (const uint16_t *)b, (uint16_t *)out, ix, total);
    else binary_low_kernel<2><<<grid, kThreads, 0, s>>>((int)op, (const uint16_t *)a, (const uint16_t *)b, (uint16_t *)out, ix, total);
    return cudaGetLastError();
}

cudaError_t unary_low(cudaStream_t s, int kind, Op op, const void *a, void *out, int64_t total) {
    if (total == 0) return cudaSuccess;
    if (kind != 1 && kind != 2) return cudaErrorInvalidValue;
    const int grid = grid_for(total, kThreads);
    if (kind == 1) unary_low_kernel<1><<<grid, kThreads, 0, s>>>((int)op, (const uint16_t *)a, (uint16_t *)out, total);
    else unary_low_kernel<2><<<grid, kThreads, 0, s>>>((int)op, (const uint16_t *)a, (uint16_t *)out, total);
    return cudaGetLastError();
}

cudaError_t argmax_rows_low(cudaStream_t s, int kind, const void *x, int64_t *out, int64_t rows, int64_t cols) {
    if (rows == 0) return cudaSuccess;
    if (kind != 1 && kind != 2) return cudaErrorInvalidValue;
    const int grid = grid_for(rows, kThreads / 32);
    if (kind == 1) argmax_low_kernel<1><<<grid, kThreads, 0, s>>>((const uint16_t *)x, out, rows, cols);
    else argmax_low_kernel<2><<<grid, kThreads, 0, s>>>((const uint16_t *)x, out, rows, cols);
    return cudaGetLastError();
}

cudaError_t row_reduce(cudaStream_t s, Op op, const float *x, float *out, int64_t rows, int64_t cols) {
    if (rows == 0) return cudaSuccess;
    row_reduce_kernel<<<grid_for(rows, kThreads / 32), kThreads, 0, s>>>((int)op, x, out, rows, cols);
    return cudaGetLastError();
}

cudaError_t full_sum(cudaStream_t s, const float *x, const Index4 &ix, int64_t total, float *out) {
    full_sum_kernel<<<1, 1024, 0, s>>>(x, ix, total, out);
    return cudaGetLastError();
}

cudaError_t argmax_rows(cudaStream_t s, const float *x, int64_t *out, int64_t rows, int64_t cols) {
    if (rows == 0) return cudaSuccess;
    const int grid = grid_for(rows, kThreads / 32);
    if ((cols & 3) == 0 && cols >= 128 && cols <= 1024 && ((uintptr_t)x & 15) == 0) {
        int chunks = (int)((cols / 4 + 31) / 32);
        if (chunks <= 1) argmax_vec_kernel<1><<<grid, kThreads, 0, s>>>(x, out, rows, (int)cols);
        else if (chunks <= 2) argmax_vec_kernel<2><<<grid, kThreads, 0, s>>>(x, out, rows, (int)cols);
        else if (chunks <= 4) argmax_vec_kernel<4><<<grid, kThreads, 0, s>>>(x, out, rows, (int)cols);
        else argmax_vec_kernel<8><<<grid, kThreads, 0, s>>>(x, out, rows, (int)cols);
    } else argmax_kernel<<<grid, kThreads, 0, s>>>(x, out, rows, cols);
    return cudaGetLastError();
}

cudaError_t softmax_rows(cudaStream_t s, const float *x, float *out, int64_t rows, int64_t cols, bool log_kind) {
    if (rows == 0) return cudaSuccess;
    const int grid = grid_for(rows, kThreads / 32);
    const bool vec = (cols & 3) == 0 && cols >= 128 && cols <= 1024 && (((uintptr_t)x | (uintptr_t)out) & 15) == 0;
#define SYN_SOFTMAX_VEC(C) do { if (log_kind) softmax_rows_vec_kernel<C, true><<<grid, kThreads, 0, s>>>(x, out, rows, (int)cols); \
                                else softmax_rows_vec_kernel<C, false><<<grid, kThreads, 0, s>>>(x, out, rows, (int)cols); } while (0)
    if (vec) {
        const int chunks = (int)((cols / 4 + 31) / 32);
        if (chunks <= 1) SYN_SOFTMAX_VEC(1); else if (chunks <= 2) SYN_SOFTMAX_VEC(2); else if (chunks <= 4) SYN_SOFTMAX_VEC(4); else SYN_SOFTMAX_VEC(8);
    } else if (log_kind) softmax_kernel<true><<<grid, kThreads, 0, s>>>(x, out, rows, cols);
    else softmax_kernel<false><<<grid, kThreads, 0, s>>>(x, out, rows, cols);
#undef SYN_SOFTMAX_VEC
    return cudaGetLastError();
}

int64_t mse_partial_count(int64_t count) {
    if (count <= 65536) return 0;                          // small inputs keep the reference's own order in one thread
    const int64_t want = (count + 4 * kMsePartialThreads * 4 - 1) / (4 * kMsePartialThreads * 4);    // at least four 16-byte groups per thread
    return want < 148 * 8 ? want : 148 * 8;
}

cudaError_t softmax_backward_rows(cudaStream_t s, const float *y, const float *g, float *out, int64_t rows, int64_t cols, bool log_kind) {
    if (rows == 0 || cols == 0) return cudaSuccess;
    const int grid = grid_for(rows, kThreads / 32);
    if (log_kind) softmax_backward_rows_kernel<true><<<grid, kThreads, 0, s>>>(y, g, out, rows, cols);
    else softmax_backward_rows_kernel<false><<<grid, kThreads, 0, s>>>(y, g, out, rows, cols);
    return cudaGetLastError();
}

cudaError_t mse(cudaStream_t s, int reduction, const float *p, const float *t, int64_t count, float *out, double *partials) {
    if (reduction == 0) {
        if (count == 0) return cudaSuccess;
        squared_error_kernel<<<grid_for(count, kThreads), kThreads, 0, s>>>(p, t, count, out);
    } else if (partials && mse_partial_count(count) > 0) {
        const int blocks = (int)mse_partial_count(count);
        mse_partial_kernel<<<blocks, kMsePartialThreads, 0, s>>>(p, t, count, partials);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return e;
        mse_final_kernel<<<1, 1024, 0, s>>>(partials, blocks, count, out, reduction == 1);
    } else {
        mse_kernel<<<1, 1024, 0, s>>>(p, t, count, out, reduction == 1);
    }
    return cudaGetLastError();
}

cudaError_t relu_backward(cudaStream_t s, const float *gate, const float *upstream, float *out, int64_t total) {
    if (total == 0) return cudaSuccess;
    bool aligned = (((uintptr_t)gate | (uintptr_t)upstream | (uintptr_t)out) & 15) == 0;
    int64_t vec = aligned ? total / 4 : 0;
    relu_backward_kernel<<<grid_for(aligned ? vec : total, kThreads), kThreads, 0, s>>>(
        (const float4 *)gate, (const float4 *)upstream, (float4 *)out, vec, gate, upstream, out, total);
    return cudaGetLastError();
}

int64_t colsum_partial_count(int64_t rows, int64_t cols) { return colsum_splits(rows, cols) * cols; }

bool colsum_can_split(const float *g, int64_t cols, int64_t pitch) {
    return (cols & 3) == 0 && (pitch & 3) == 0 && ((uintptr_t)g & 15) == 0;
}

cudaError_t colsum(cudaStream_t s, const float *g, int64_t rows, int64_t cols, double *partials, float *out,
                   float *plane_hi, float *plane_lo, int64_t pitch) {
    if (cols == 0) return cudaSuccess;
    int64_t splits = colsum_splits(rows, cols);
    int64_t rows_per = (rows + splits - 1) / splits;
    dim3 grid((unsigned)((cols + 127) / 128), (unsigned)splits);
    if (plane_hi) {
        if (!colsum_can_split(g, cols, pitch) || !plane_lo) return cudaErrorInvalidValue;
        colsum_partial_kernel<true><<<grid, kColsumRows * 32, 0, s>>>(g, rows, cols, rows_per, partials, plane_hi, plane_lo, pitch);
    } else {
        colsum_partial_kernel<false><<<grid, kColsumRows * 32, 0, s>>>(g, rows, cols, rows_per, partials, nullptr, nullptr, 0);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    if (cols < 128 && splits >= 64) colsum_final_narrow_kernel<<<(unsigned)((cols + 7) / 8), 256, 0, s>>>(partials, splits, cols, out);
    else colsum_final_kernel<<<(unsigned)((cols + 255) / 256), 256, 0, s>>>(partials, splits, cols, out);
    return cudaGetLastError();
}

// ---- column sums without any allocation ----------------------------------------------------------
// Scratch for callers that cannot allocate device memory.  In host code the array's name is only a
// stand-in for the symbol, never a device address, so the address is looked up once per device
// (with that device current) and the kernels receive the looked-up pointer.
static __device__ __align__(256) double g_colsum_static_partials[kStaticColsumPartials];
static double *g_colsum_static_address[64];
static std::mutex g_colsum_static_mutex;

cudaError_t colsum_static(cudaStream_t s, int device, const float *g, int64_t rows, int64_t cols, float *out) {
    if (device < 0 || device >= 64) return cudaErrorInvalidDevice;
    if (cols == 0) return cudaSuccess;
    if (colsum_partial_count(rows, cols) > kStaticColsumPartials) return cudaErrorInvalidValue;
    double *partials;
    {
        std::lock_guard<std::mutex> lock(g_colsum_static_mutex);
        if (!g_colsum_static_address[device]) {
            void *address = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&address, g_colsum_static_partials);
            if (e != cudaSuccess) return e;
            g_colsum_static_address[device] = static_cast<double *>(address);
        }
        partials = g_colsum_static_address[device];
    }
    // phase 1 writes every partial that phase 2 reads, so nothing of an earlier call survives and
    // nothing has to be cleared first
    return colsum(s, g, rows, cols, partials, out, nullptr, nullptr, 0);
}

cudaError_t cross_entropy(cudaStream_t s, const float *logits, DType label_type, const void *labels, const float *seed,
                          int64_t rows, int64_t cols, float *row_loss, float *loss_out, float *grad_out, int64_t *argmax_out, int *error_word,
                          int sum_only, int has_ignore, int64_t ignore, int scale_mode, float *active_scratch) {
    if (rows == 0 || cols == 0) return cudaErrorInvalidValue;
    if (scale_mode < 0 || scale_mode > 2 || (scale_mode == 2 && grad_out && !seed)) return cudaErrorInvalidValue;
    // the MEAN gradient under an ignore index divides by the rows that are left: counted first
    const float *divisor = nullptr;
    if (has_ignore && grad_out && scale_mode == 0) {
        if (!active_scratch) return cudaErrorInvalidValue;
        if (label_type == DType::I32) count_active_kernel<int32_t><<<1, 1024, 0, s>>>(labels, (long long)ignore, rows, active_scratch);
        else count_active_kernel<int64_t><<<1, 1024, 0, s>>>(labels, (long long)ignore, rows, active_scratch);
        cudaError_t ce = cudaGetLastError();
        if (ce != cudaSuccess) return ce;
        divisor = active_scratch;
    }
    int grid = grid_for(rows, kThreads / 32);
    bool vec = (cols & 3) == 0 && cols >= 128 && cols <= 1024 && (((uintptr_t)logits | (uintptr_t)grad_out) & 15) == 0;
    bool i32 = label_type == DType::I32;
#define SYN_CE_ARGS <<<grid, kThreads, 0, s>>>(logits, labels, seed, rows, (int)cols, row_loss, grad_out, argmax_out, error_word, has_ignore, (long long)ignore, scale_mode, divisor)
#define SYN_CE_VEC2(C, L) do { if (grad_out && argmax_out) ce_rows_vec_kernel<C, L, true, true> SYN_CE_ARGS; \
                               else if (grad_out) ce_rows_vec_kernel<C, L, true, false> SYN_CE_ARGS; \
                               else if (argmax_out) ce_rows_vec_kernel<C, L, false, true> SYN_CE_ARGS; \
                               else ce_rows_vec_kernel<C, L, false, false> SYN_CE_ARGS; } while (0)
#define SYN_CE_VEC(C) do { if (i32) SYN_CE_VEC2(C, int32_t); else SYN_CE_VEC2(C, int64_t); } while (0)
    if (vec) {
        int chunks = (int)((cols / 4 + 31) / 32);
        if (chunks <= 1) SYN_CE_VEC(1); else if (chunks <= 2) SYN_CE_VEC(2); else if (chunks <= 4) SYN_CE_VEC(4); else SYN_CE_VEC(8);
    } else if (i32) ce_rows_generic_kernel<int32_t><<<grid, kThreads, 0, s>>>(logits, labels, seed, rows, cols, row_loss, grad_out, argmax_out, error_word, has_ignore, (long long)ignore, scale_mode, divisor);
    else ce_rows_generic_kernel<int64_t><<<grid, kThreads, 0, s>>>(logits, labels, seed, rows, cols, row_loss, grad_out, argmax_out, error_word, has_ignore, (long long)ignore, scale_mode, divisor);
#undef SYN_CE_VEC
#undef SYN_CE_VEC2
#undef SYN_CE_ARGS
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || !loss_out) return e;
    if (!has_ignore) mean_kernel<<<1, 1024, 0, s>>>(row_loss, rows, loss_out, !sum_only);
    else if (i32) mean_active_kernel<int32_t><<<1, 1024, 0, s>>>(row_loss, labels, (long long)ignore, rows, loss_out, !sum_only);
    else mean_active_kernel<int64_t><<<1, 1024, 0, s>>>(row_loss, labels, (long long)ignore, rows, loss_out, !sum_only);
    return cudaGetLastError();
}

cudaError_t dense_cross_entropy(cudaStream_t s, const float *logits, const float *target, int64_t rows, int64_t cols,
                                float *row_loss, float *loss_out, int sum_only) {
    if (rows == 0 || cols == 0) return cudaErrorInvalidValue;
    const int grid = grid_for(rows, kThreads / 32);
    const bool vec = (cols & 3) == 0 && cols >= 128 && cols <= 1024 && (((uintptr_t)logits | (uintptr_t)target) & 15) == 0;
    if (vec) {
        const int chunks = (int)((cols / 4 + 31) / 32);
        if (chunks <= 1) dense_ce_rows_vec_kernel<1><<<grid, kThreads, 0, s>>>(logits, target, rows, (int)cols, row_loss);
        else if (chunks <= 2) dense_ce_rows_vec_kernel<2><<<grid, kThreads, 0, s>>>(logits, target, rows, (int)cols, row_loss);
        else if (chunks <= 4) dense_ce_rows_vec_kernel<4><<<grid, kThreads, 0, s>>>(logits, target, rows, (int)cols, row_loss);
        else dense_ce_rows_vec_kernel<8><<<grid, kThreads, 0, s>>>(logits, target, rows, (int)cols, row_loss);
    } else dense_ce_rows_kernel<<<grid, kThreads, 0, s>>>(logits, target, rows, cols, row_loss);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || !loss_out) return e;
    mean_kernel<<<1, 1024, 0, s>>>(row_loss, rows, loss_out, !sum_only);
    return cudaGetLastError();
}

cudaError_t dense_cross_entropy_backward(cudaStream_t s, const float *logits, const float *target, const float *seed, int64_t rows, int64_t cols,
                                         float *grad, int scale_mode) {
    if (rows == 0 || cols == 0) return cudaErrorInvalidValue;
    if (scale_mode < 0 || scale_mode > 2 || (scale_mode == 2 && !seed)) return cudaErrorInvalidValue;
    const int grid = grid_for(rows, kThreads / 32);
    const bool vec = (cols & 3) == 0 && cols >= 128 && cols <= 1024 && (((uintptr_t)logits | (uintptr_t)target | (uintptr_t)grad) & 15) == 0;
    if (vec) {
        const int chunks = (int)((cols / 4 + 31) / 32);
        if (chunks <= 1) dense_ce_grad_rows_vec_kernel<1><<<grid, kThreads, 0, s>>>(logits, target, seed, rows, (int)cols, grad, scale_mode);
        else if (chunks <= 2) dense_ce_grad_rows_vec_kernel<2><<<grid, kThreads, 0, s>>>(logits, target, seed, rows, (int)cols, grad, scale_mode);
        else if (chunks <= 4) dense_ce_grad_rows_vec_kernel<4><<<grid, kThreads, 0, s>>>(logits, target, seed, rows, (int)cols, grad, scale_mode);
        else dense_ce_grad_rows_vec_kernel<8><<<grid, kThreads, 0, s>>>(logits, target, seed, rows, (int)cols, grad, scale_mode);
    } else dense_ce_grad_rows_kernel<<<grid, kThreads, 0, s>>>(logits, target, seed, rows, cols, grad, scale_mode);
    return cudaGetLastError();
}

cudaError_t sgd_step(cudaStream_t s, const TensorSlot *slots, int slot_count, const SgdArgs &args, int *error_word) {
    return launch_slots(s, sgd_kernel, slots, slot_count, args, error_word);
}
cudaError_t adam_step(cudaStream_t s, const TensorSlot *slots, int slot_count, const AdamArgs &args, int *error_word) {
    return launch_slots(s, adam_kernel, slots, slot_count, args, error_word);
}
cudaError_t clear_pending(cudaStream_t s, const TensorSlot *slots, int slot_count, int *error_word) {
    return launch_slots(s, clear_pending_kernel, slots, slot_count, NoArgs{}, error_word);
}
cudaError_t accumulate_gradients(cudaStream_t s, const TensorSlot *slots, int slot_count, int sequence, int *failed_sequence, int *error_word) {
    AccumulateArgs args{sequence, failed_sequence};
    cudaError_t e = launch_slots(s, accumulate_kernel<false>, slots, slot_count, args, error_word);
    if (e != cudaSuccess) return e;
    return launch_slots(s, accumulate_kernel<true>, slots, slot_count, args, error_word);
}

}  // namespace kern
}  // namespace syn
