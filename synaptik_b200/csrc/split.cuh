// hi / lo split of a binary32 value for the 3xTF32 products: hi = tf32(x), lo = tf32(x - hi).
// x - hi is exact in binary32, so hi + lo carries 22 significand bits of x.
#pragma once
#include <cstdint>

namespace syn {
namespace kern {

__device__ __forceinline__ float to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}
__device__ __forceinline__ bool finite_bits(float x) { return (__float_as_uint(x) & 0x7f800000u) != 0x7f800000u; }
__device__ __forceinline__ void split_value(float x, float &hi, float &lo) {
    float h = to_tf32(x);
    if (!finite_bits(h)) {
        if (!finite_bits(x)) { hi = x; lo = 0.0f; return; }         // inf / NaN pass through the hi plane only
        h = __uint_as_float(__float_as_uint(x) & 0xffffe000u);      // rounding up would overflow: truncate instead
    }
    hi = h;
    lo = to_tf32(__fsub_rn(x, h));
}

}  // namespace kern
}  // namespace syn
