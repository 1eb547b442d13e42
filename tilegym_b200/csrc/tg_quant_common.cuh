// Element-wise core of the 8-bit quantisers: bytes = cast(clamp(x / s, min, max)), identical to what an IEEE
// (round-to-nearest) division followed by the cast gives, at a fraction of the instruction count.
//
// Two costs bound these streaming kernels before HBM does.  div.rn.f32 is 10-15 instructions per element, and
// the float -> fp8 conversion unit converts about one lane (two values) per clock per SM sub-partition, so there
// is room for exactly one two-wide conversion per pair of elements and nothing more.  Hence: the group's
// reciprocal r = RN(1 / s) is computed once, a = x * r is within 1.2e-7 (relative, two ulps) of the true
// quotient Q, and cast(a) == cast(RN(Q)) unless a lies within a few ulps of one of the TARGET format's
// rounding boundaries - a test on the bits of a, no conversion needed.  Only those elements (about one in
// 10^5, plus the target's subnormal range, where the boundaries sit elsewhere) are redone with __fdiv_rn.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include <type_traits>

namespace tg {

enum Q8Kind : int { kQ8E4M3 = 0, kQ8E5M2 = 1, kQ8Int8 = 2 };

// Programmatic dependent launch, primary side: a kernel launched behind this one with programmatic stream
// serialization (the GEMMs are) may be scheduled from now on and run the part in front of its griddepcontrol.wait -
// barrier set-up, TMEM allocation, streaming weights declared static - while the quantiser still works; what it reads
// of the quantiser's output it reads after that wait, which returns when this grid has completed.
__device__ __forceinline__ void q8_allow_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// The reciprocal path needs a scale whose reciprocal and products stay in the normal range; the elements of a
// group whose scale is outside it all take __fdiv_rn.
__device__ __forceinline__ bool q8_scale_is_tame(float s) { return s > 1e-20f && s < 1e20f; }

// Smallest power of two >= max(|s|, 1e-10): ceil(log2) read off the exponent and mantissa bits, so the
// result does not depend on a log2 implementation.
__device__ __forceinline__ float round_up_pow2(float s) {
  s = fmaxf(fabsf(s), 1e-10f);
  const uint32_t b = __float_as_uint(s);
  const uint32_t exp_bits = (b & 0x7f800000u) + ((b & 0x007fffffu) ? 0x00800000u : 0u);
  return __uint_as_float(exp_bits);
}

// May cast(a) differ from cast(q) for some q within 4 ulps of a?
template <int KIND>
__device__ __forceinline__ bool q8_unsafe(float a) {
  if constexpr (KIND == kQ8Int8) {
    // truncation changes at integers; beyond +-130 the clamp decides
    const float rn = (a + 12582912.f) - 12582912.f;  // nearest integer for |a| < 2^22
    return a != 0.f && fabsf(a) < 130.f && fabsf(a - rn) <= fabsf(a) * 4.8e-7f;
  } else {
    // round-to-nearest-even to 3 (e4m3) or 2 (e5m2) mantissa bits changes at the midpoints, where the
    // dropped fp32 mantissa bits read 100...0; below the target's normal range the boundaries sit elsewhere
    constexpr int kDrop = (KIND == kQ8E4M3) ? 20 : 21;
    constexpr uint32_t kMask = (1u << kDrop) - 1u, kMid = 1u << (kDrop - 1);
    constexpr uint32_t kTinyBits = (KIND == kQ8E4M3) ? 0x3d000000u : 0x39000000u;  // 2^-5, 2^-13: 2 x smallest normal
    const uint32_t b = __float_as_uint(a) & 0x7fffffffu;
    return ((b - (kMid - 4u)) & kMask) <= 8u || (b - 1u) < (kTinyBits - 1u);  // zero is exact: excluded
  }
}

template <int KIND>
__device__ __forceinline__ uint32_t q8_cast2(float lo, float hi, float qmin, float qmax) {
  if constexpr (KIND == kQ8Int8) {
    lo = fminf(fmaxf(lo, qmin), qmax);
    hi = fminf(fmaxf(hi, qmin), qmax);
    return (static_cast<uint32_t>(__float2int_rz(lo)) & 0xffu) | ((static_cast<uint32_t>(__float2int_rz(hi)) & 0xffu) << 8);
  } else {
    // the fp8 casts saturate to the largest finite value by themselves (the clamp) and keep NaN
    return static_cast<uint32_t>(
        __nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, KIND == kQ8E4M3 ? __NV_E4M3 : __NV_E5M2));
  }
}

// x / s for two neighbouring elements, correctly rounded, from the group's reciprocal r = RN(1 / s) with three
// packed FMA-pipe instructions and no test: a = x r is within two ulps of the quotient, e = x - a s is exact in
// an FMA, and a + e r is the quotient to ~2^-46 before its single rounding (Markstein's correction step).  For
// 16-bit inputs and scales of the form RN(amax / qmax) the result has been compared with div.rn for EVERY
// (amax, x) pair (tg_selftest_quant16: 2^31 quotients per input type and target format); callers use it for
// those only.  e is +0 whenever the residual vanishes, which would turn x = -0 into +0: x's sign bit is put back
// (a no-op for every other x, since r > 0).
__device__ __forceinline__ float2 q8_quot2(float2 x, float s, float r) {
  const float2 r2 = make_float2(r, r);
  const float2 a = __fmul2_rn(x, r2);
  const float2 e = __ffma2_rn(a, make_float2(-s, -s), x);
  float2 q = __ffma2_rn(e, r2, a);
  q.x = __uint_as_float(__float_as_uint(q.x) | (__float_as_uint(x.x) & 0x80000000u));
  q.y = __uint_as_float(__float_as_uint(q.y) | (__float_as_uint(x.y) & 0x80000000u));
  return q;
}

// amax / qmax (qmax = 448, 57344 or 127) the same way: c = RN(1 / qmax).  Exact for every 16-bit amax whose
// quotient is a normal number (checked by the same self-test); smaller ones take div.rn.
__device__ __forceinline__ float q8_scale_from_amax(float amax, float qmax, float c) {
  if (amax < 1e-30f) return __fdiv_rn(amax, qmax);
  const float q = amax * c;
  return __fmaf_rn(__fmaf_rn(-q, qmax, amax), c, q);
}

// |x| maximum of two packed 16-bit pairs, element-wise (NaN operands are ignored, like fmaxf).
template <typename T>
__device__ __forceinline__ uint32_t absmax_pairs(uint32_t a, uint32_t b) {
  if constexpr (std::is_same<T, __half>::value) {
    const __half2 m = __hmax2(__habs2(*reinterpret_cast<const __half2*>(&a)), __habs2(*reinterpret_cast<const __half2*>(&b)));
    return *reinterpret_cast<const uint32_t*>(&m);
  } else {
    const __nv_bfloat162 m = __hmax2(__habs2(*reinterpret_cast<const __nv_bfloat162*>(&a)),
                                     __habs2(*reinterpret_cast<const __nv_bfloat162*>(&b)));
    return *reinterpret_cast<const uint32_t*>(&m);
  }
}

template <typename T>
__device__ __forceinline__ float2 unpack_pair(uint32_t w) {
  if constexpr (std::is_same<T, __half>::value) return __half22float2(*reinterpret_cast<const __half2*>(&w));
  else return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));  // bf16 -> fp32 is a shift
}

// Two neighbouring elements -> two bytes (x0 in the low byte).
template <int KIND>
__device__ __forceinline__ uint32_t q8_pair(float x0, float x1, float s, float r, bool tame, float qmin, float qmax) {
  float a0 = x0 * r, a1 = x1 * r;
  if (!tame || q8_unsafe<KIND>(a0) || q8_unsafe<KIND>(a1)) {
    a0 = __fdiv_rn(x0, s);
    a1 = __fdiv_rn(x1, s);
  }
  return q8_cast2<KIND>(a0, a1, qmin, qmax);
}

}  // namespace tg
