// UE8M0 / E4M3 / E2M1 encoding helpers shared by the quantisation kernels and by GEMM epilogues that
// quantise their own output.  Contract (bit-exact): deepgemm/src/golden.rs:142-241.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace dg {

// ------------------------------------------------------------------------- device helpers
// amax -> biased UE8M0 exponent (golden.rs:211-241): round amax/qmax up to a power of two.
template <bool FP4>
__device__ __forceinline__ uint32_t ue8m0_exp(float amax) {
    constexpr uint32_t kQMaxMant = FP4 ? (0x40u << 16) : (0x60u << 16);
    constexpr uint32_t kQExp = FP4 ? 2u : 8u;
    constexpr uint32_t kMinExp = FP4 ? 1u : 105u;
    uint32_t rounded = (__float_as_uint(amax) + 0x7fffffu - kQMaxMant) >> 23;
    return max(rounded, kMinExp + kQExp) - kQExp;
}

// Four scaled floats -> four E4M3 bytes (element 0 in the low byte), RNE, saturating.
// NaN encodes as a signed zero code, like the golden model's grid search (golden.rs:142-189); its
// sign is the input's (`src`): the multiplication by the scale returns the canonical positive NaN.
__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d, const float4& src) {
    uint16_t lo, hi;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
    uint32_t r = (uint32_t)lo | ((uint32_t)hi << 16);
    // The saturating conversion never produces 0x7f / 0xff for a number (the largest finite code is
    // 0x7e), so a byte with all seven low bits set marks a NaN input: a rare, single test.
    if (((r & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u) {
        if (a != a) r = (r & 0xffffff00u) | ((__float_as_uint(src.x) >> 31) << 7);
        if (b != b) r = (r & 0xffff00ffu) | ((__float_as_uint(src.y) >> 31) << 15);
        if (c != c) r = (r & 0xff00ffffu) | ((__float_as_uint(src.z) >> 31) << 23);
        if (d != d) r = (r & 0x00ffffffu) | ((__float_as_uint(src.w) >> 31) << 31);
    }
    return r;
}
// Two scaled floats -> one byte of two E2M1 nibbles (first element in the low nibble).
__device__ __forceinline__ uint32_t cvt_e2m1x2(float a, float b, float src_a, float src_b) {
    uint16_t r;
    asm("{ .reg .b8 t;\n cvt.rn.satfinite.e2m1x2.f32 t, %2, %1;\n mov.b16 %0, {t, 0}; }" : "=h"(r) : "f"(a), "f"(b));
    uint32_t v = r;
    if (a != a) v = (v & 0xf0u) | ((__float_as_uint(src_a) >> 31) << 3);
    if (b != b) v = (v & 0x0fu) | ((__float_as_uint(src_b) >> 31) << 7);
    return v;
}

__device__ __forceinline__ float amax4(const float4& v) {
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}

}  // namespace dg
