// 16-bit storage types (BFLOAT16 / FLOAT16) with a FLOAT32 working type: the reference keeps such tensors
// as raw 16-bit patterns, widens every operand to FLOAT32, computes there and narrows each node's result
// once (CpuScalarReferenceKernel.java:93-115).  KIND 1 = BFLOAT16, 2 = FLOAT16.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

#include "activation.cuh"

namespace syn {
namespace kern {

template <int KIND> __device__ __forceinline__ float low_decode(uint16_t bits) {
    if constexpr (KIND == 1) return __uint_as_float((uint32_t)bits << 16);
    else return __half2float(__ushort_as_half(bits));
}
// Round to nearest even.  BFLOAT16: any NaN becomes 0x7FC0 and the discarded 16 bits decide the rounding
// (BFloat16Bits.java:17-29); FLOAT16: any NaN becomes 0x7E00, otherwise the IEEE conversion (Float16Bits.java).
template <int KIND> __device__ __forceinline__ uint16_t low_encode(float x) {
    if constexpr (KIND == 1) {
        uint16_t rounded;               // the hardware conversion rounds to nearest even; only its NaN pattern differs
        asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(rounded) : "f"(x));
        return x != x ? (uint16_t)0x7FC0 : rounded;
    } else {
        if (x != x) return 0x7E00;
        return __half_as_ushort(__float2half_rn(x));
    }
}
template <int KIND> __device__ __forceinline__ float low_round(float x) { return low_decode<KIND>(low_encode<KIND>(x)); }

// FLOAT32 working result of an activation on an exactly decoded low input, before the one narrowing.
// SIGMOID, SILU and both GELUs are FLOAT32 composites, every product, sum and quotient a binary32 rounding,
// the elementary function taken in binary64 and narrowed at once, -inf giving -0 except for SIGMOID
// (CpuScalarReferenceKernel.lowActivation, :1753-1775); RELU and TANH as for FLOAT32 values (:1722-1742).
__device__ __forceinline__ float low_activation_value(int act, float x) {
    switch ((Op)act) {
        case Op::RELU: return relu_value(x);
        case Op::TANH: return tanh_value(x);
        case Op::SIGMOID: {
            const float e = (float)exp((double)(x >= 0.0f ? -x : x));
            return __fdiv_rn(x >= 0.0f ? 1.0f : e, __fadd_rn(1.0f, e));
        }
        case Op::SILU: {
            if (x == -CUDART_INF_F) return -0.0f;
            const float e = (float)exp((double)(x >= 0.0f ? -x : x));
            return __fdiv_rn(x >= 0.0f ? x : __fmul_rn(x, e), __fadd_rn(1.0f, e));
        }
        case Op::GELU: {
            if (x == -CUDART_INF_F) return -0.0f;
            const float root = 1.41421354f;                         // (float) sqrt(2.0f)
            const float inner = (float)erf((double)__fdiv_rn(x, root));
            return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, inner));
        }
        case Op::GELU_TANH: {
            if (x == -CUDART_INF_F) return -0.0f;
            const float cube = __fmul_rn(__fmul_rn(x, x), x);
            const float scale = 0.79788452f;                        // (float) sqrt(2.0f / (float) pi) = 0x3F4C4229
            const float argument = __fmul_rn(scale, __fadd_rn(x, __fmul_rn(0.044715f, cube)));
            const float inner = (float)tanh((double)argument);
            return __fmul_rn(__fmul_rn(0.5f, x), __fadd_rn(1.0f, inner));
        }
        default: return x;
    }
}

}  // namespace kern
}  // namespace syn
