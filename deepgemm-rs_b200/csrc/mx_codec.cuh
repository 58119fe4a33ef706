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

// 32 well-mixed bits from a 64-bit element index and a seed (the finaliser of MurmurHash3 over the folded
// index); the stochastic quantiser's only source of randomness.
__host__ __device__ __forceinline__ uint32_t hash_u32(uint64_t idx, uint32_t seed) {
    uint32_t x = (uint32_t)idx * 0x9E3779B9u + (uint32_t)(idx >> 32) * 0x7F4A7C15u + seed;
    x ^= x >> 16; x *= 0x85EBCA6Bu;
    x ^= x >> 13; x *= 0xC2B2AE35u;
    x ^= x >> 16;
    return x;
}
// Stochastic rounding of a scaled value (|v| <= 448) onto the E4M3 grid: returns the chosen grid value
// (exactly representable, so the RNE conversion that follows encodes it unchanged).  lo = the grid
// value at or below |v|, one grid step = 2^-9 below 2^-6 (subnormals) and 2^(exponent - 3) above; the
// value goes up when the top 24 bits of `rnd`, read as a fraction, lie below (|v| - lo) / step.
// Every operation is exact in f32.  NaN passes through (it encodes as a signed zero afterwards).
__host__ __device__ __forceinline__ float stochastic_e4m3_value(float v, uint32_t rnd) {
    union { float f; uint32_t u; } in, t;
    in.f = v;
    const uint32_t sign = in.u & 0x80000000u, mag_bits = in.u & 0x7fffffffu;
    if (mag_bits > 0x7f800000u) return v;                 // NaN
    t.u = mag_bits;
    const float a = t.f;
    if (a >= 448.f) { t.u = sign | 0x43e00000u; return t.f; }   // the scale keeps |v| <= 448; clamp anyway
    uint32_t e = mag_bits >> 23;                          // biased exponent
    if (e < 121u) e = 121u;                               // below 2^-6 the grid step stays 2^-9
    t.u = (e - 3u) << 23;  const float step = t.f;
    t.u = (257u - e) << 23; const float inv_step = t.f;
    const float units = a * inv_step;                     // exact: a power-of-two scaling
    const float fl = (float)(uint32_t)units;              // floor, units < 16
    const float frac = units - fl;
    const float u = (float)(rnd >> 8) * (1.0f / 16777216.0f);
    const float r = (u < frac ? fl + 1.0f : fl) * step;
    t.f = r;
    t.u |= sign;
    return t.f;
}

// silu(g) * u in f32, defined operation by operation so that the CPU checker can state the same function
// and the re-quantised codes agree bit for bit; every step is a correctly rounded f32 operation on the FMA
// pipe or an integer operation, none goes through the special-function unit (an eighth of the lanes):
//   x = -g clamped to [-87, 87]
//   t = fma(x, log2 e, 1.5 * 2^23): the low mantissa bits of t hold n = round(x * log2 e); nf = t - 1.5 * 2^23
//   f = x - nf * ln 2 (two-step Cody-Waite), p = degree-6 Taylor polynomial of exp(f) in Horner form
//   2^n = bits (t << 23) + 0x3f800000;  d = fma(p, 2^n, 1) = 1 + exp(-g)   (p * 2^n is within about 1 ulp of expf)
//   r = 1 / d by three Newton steps r += r * (1 - d * r) from the seed bits 0x7ef311c7 - bits(d)
//       (5 % off; 4e-11 after three steps, so r is d's reciprocal to the last bit or the one beside it)
//   result (g * r) * u
constexpr float kSwLog2e = 1.44269502162933349609375f;
constexpr float kSwMagic = 12582912.0f;
constexpr float kSwLn2Hi = -0.693145751953125f;
constexpr float kSwLn2Lo = -1.428606765330187045037746429443359375e-06f;
__device__ __forceinline__ float swiglu_value(float g, float u) {
    const float x = fminf(fmaxf(-g, -87.0f), 87.0f);
    const float t = fmaf(x, kSwLog2e, kSwMagic);
    const float n = t - kSwMagic;
    float f = fmaf(n, kSwLn2Hi, x);
    f = fmaf(n, kSwLn2Lo, f);
    float p = fmaf(f, 1.0f / 720.0f, 1.0f / 120.0f);
    p = fmaf(p, f, 1.0f / 24.0f);
    p = fmaf(p, f, 1.0f / 6.0f);
    p = fmaf(p, f, 0.5f);
    p = fmaf(p, f, 1.0f);
    p = fmaf(p, f, 1.0f);
    const float d = fmaf(p, __uint_as_float((__float_as_uint(t) << 23) + 0x3f800000u), 1.0f);
    float r = __uint_as_float(0x7ef311c7u - __float_as_uint(d));
#pragma unroll
    for (int i = 0; i < 3; ++i) r = fmaf(r, fmaf(-d, r, 1.0f), r);
    return g * r * u;
}

// The same function for two elements at once: every multiply, add and fused multiply-add is a packed f32x2
// instruction (sm_100: two lanes per instruction, each rounded as its scalar counterpart, so the results are the
// same bit for bit); the clamp and the two integer steps stay scalar.  -d is formed directly (p * -2^n - 1,
// the mirror image of d, rounding included), so that the Newton steps need no negation.
__device__ __forceinline__ uint64_t f32x2(float lo, float hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f32x2_get(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// a compile-time constant in both halves: an immediate 64-bit operand, no register pair to fill
__host__ __device__ constexpr uint64_t splat2(float v) { return (uint64_t)__builtin_bit_cast(uint32_t, v) * 0x100000001ull; }
__device__ __forceinline__ void swiglu_value2(float g0, float g1, float u0, float u1, float& r0, float& r1) {
    const float x0 = fminf(fmaxf(-g0, -87.0f), 87.0f), x1 = fminf(fmaxf(-g1, -87.0f), 87.0f);
    const uint64_t x = f32x2(x0, x1);
    const uint64_t t = fma2(x, splat2(kSwLog2e), splat2(kSwMagic));
    const uint64_t n = add2(t, splat2(-kSwMagic));
    uint64_t f = fma2(n, splat2(kSwLn2Hi), x);
    f = fma2(n, splat2(kSwLn2Lo), f);
    uint64_t p = fma2(f, splat2(1.0f / 720.0f), splat2(1.0f / 120.0f));
    p = fma2(p, f, splat2(1.0f / 24.0f));
    p = fma2(p, f, splat2(1.0f / 6.0f));
    p = fma2(p, f, splat2(0.5f));
    p = fma2(p, f, splat2(1.0f));
    p = fma2(p, f, splat2(1.0f));
    float t0, t1;
    f32x2_get(t, t0, t1);
    const uint64_t nscale = f32x2(__uint_as_float((__float_as_uint(t0) << 23) + 0xbf800000u),
                                  __uint_as_float((__float_as_uint(t1) << 23) + 0xbf800000u));      // -2^n
    const uint64_t nd = fma2(p, nscale, splat2(-1.0f));                                             // -(1 + exp(-g))
    float nd0, nd1;
    f32x2_get(nd, nd0, nd1);
    uint64_t r = f32x2(__uint_as_float(0xfef311c7u - __float_as_uint(nd0)), __uint_as_float(0xfef311c7u - __float_as_uint(nd1)));
#pragma unroll
    for (int i = 0; i < 3; ++i) r = fma2(r, fma2(nd, r, splat2(1.0f)), r);
    f32x2_get(mul2(mul2(f32x2(g0, g1), r), f32x2(u0, u1)), r0, r1);
}

__device__ __forceinline__ float amax4(const float4& v) {
    return fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
}

}  // namespace dg
