// Activation functions on FLOAT32 values, shared by the element-wise kernel and the GEMM epilogues so
// that an activation fused into a product gives the very bits the separate pass would.
#pragma once
#include <cstdint>
#include <math_constants.h>

#include "program.hpp"

namespace syn {
namespace kern {

// Math.max(x, +0.0f): NaN stays NaN, -0 -> +0
__device__ __forceinline__ float relu_value(float x) { return x != x ? x : (x > 0.0f ? x : 0.0f); }

// TANH and SIGMOID follow the reference's FLOAT32 path: the elementary function in binary64, one
// narrowing to binary32 (CpuScalarReferenceKernel.java:1729-1742; sigmoid as 1 / (1 + exp(-x)) for
// x >= 0 and exp(x) / (1 + exp(x)) below, CpuScalarEmitter.java:429-439).  The device's binary64 tanh
// and exp are within 1-2 ulp of binary64, so the narrowed result differs from (float)StrictMath only on
// rounding ties of probability ~2^-28.
__device__ __forceinline__ float tanh_value(float x) { return (float)tanh((double)x); }
__device__ __forceinline__ float sigmoid_value(float x) {
    const double v = (double)x;
    if (v < 0.0 || v != v) { const double e = exp(v); return (float)(e / (1.0 + e)); }
    return (float)(1.0 / (1.0 + exp(-v)));
}

// SILU, CpuScalarReferenceKernel.java:1236-1241: -inf gives -0; x / (1 + exp(-x)) for x >= 0,
// x * exp(x) / (1 + exp(x)) below (and for NaN), in binary64, one narrowing.
__device__ __forceinline__ float silu_value(float x) {
    const double v = (double)x;
    if (v == -CUDART_INF) return -0.0f;
    if (v >= 0.0) return (float)(v / (1.0 + exp(-v)));
    const double e = exp(v);
    return (float)(v * e / (1.0 + e));
}

// Tanh-approximated GELU, CpuScalarReferenceKernel.java:1224-1229: -inf gives -0; otherwise
// 0.5 * x * (1 + tanh(sqrt(2 / pi) * (x + 0.044715 * x^3))) in binary64, one narrowing.
__device__ __forceinline__ float gelu_tanh_value(float x) {
    const double v = (double)x;
    if (v == -CUDART_INF) return -0.0f;
    const double cube = v * v * v;
    return (float)(0.5 * v * (1.0 + tanh(sqrt(2.0 / 3.14159265358979323846) * (v + 0.044715 * cube))));
}

// ERF and the exact GELU on FLOAT32 (CpuScalarEmitter.java:353-366,441-452): the value widened to
// binary64, erf (the reference's rational approximation is accurate to binary64 rounding, returns
// the signed zero unchanged and +-1 from |x| = 6 on, as the library function rounds to), for GELU
// 0.5 * x * (1 + erf(x / sqrt(2))) with -inf giving -0, then one narrowing.
__device__ __forceinline__ float erf_value(float x) { return (float)erf((double)x); }
__device__ __forceinline__ float gelu_value(float x) {
    const double v = (double)x;
    if (v == -CUDART_INF) return -0.0f;
    return (float)(0.5 * v * (1.0 + erf(v / sqrt(2.0))));
}

// One value through the activation `act` (an Op wire code; 0 leaves the value as it is).
__device__ __forceinline__ float activation_value(int act, float x) {
    switch ((Op)act) {
        case Op::RELU: return relu_value(x);
        case Op::TANH: return tanh_value(x);
        case Op::SIGMOID: return sigmoid_value(x);
        case Op::SILU: return silu_value(x);
        case Op::GELU_TANH: return gelu_tanh_value(x);
        case Op::GELU: return gelu_value(x);
        default: return x;
    }
}

}  // namespace kern
}  // namespace syn
