// Arithmetic shared by the quantizer kernels and by GEMM epilogues that quantise their output: exact
// fp32 division by a per-block constant, the narrow-format conversions, the swizzled scale-factor
// offset, and the NVFP4 block encoder.  Results equal the torch reference bit for bit:
//   * quotients are correctly rounded fp32 divisions: one correctly rounded reciprocal per block and
//     two FMA residual corrections per element (Markstein: a faithful quotient corrected once with an
//     exactly computed residual and a correctly rounded reciprocal is the correctly rounded quotient;
//     the first correction makes the estimate faithful, the second makes it exact);
//   * narrow formats come from the cvt.rn.satfinite instructions, which round to nearest even exactly
//     like the reference's casts and threshold chains.
#pragma once

#include "gnk_common.cuh"

namespace gnk {

// x / d for d > 0, given r = __frcp_rn(d).  Correctly rounded when the quotient is far
// from overflow and x is not within 2^-100 of zero (then the result only feeds a
// rounding to zero); `safe` = false takes the plain IEEE division instead.
__device__ __forceinline__ float divide_exact(float x, float d, float r, bool safe) {
  if (!safe) return __fdiv_rn(x, d);
  float q = __fmul_rn(x, r);
  float e = __fmaf_rn(-d, q, x);
  q = __fmaf_rn(e, r, q);
  e = __fmaf_rn(-d, q, x);
  q = __fmaf_rn(e, r, q);
  return copysignf(q, x);  // x = -0 must stay -0 (the packers copy the sign bit)
}

// The same correction chain on two quotients at once (packed f32x2 instructions round each lane
// exactly like their scalar forms, so the results are the same bits at half the issue slots).
// nd2 = (-d, -d), r2 = (r, r).
__device__ __forceinline__ void divide_exact_pair(float& a, float& b, uint64_t nd2, uint64_t r2) {
  const uint64_t x2 = f2_pack(a, b);
  uint64_t q = f2_mul(x2, r2);
  uint64_t e = f2_fma(nd2, q, x2);
  q = f2_fma(e, r2, q);
  e = f2_fma(nd2, q, x2);
  q = f2_fma(e, r2, q);
  float q0, q1;
  f2_unpack(q, q0, q1);
  a = copysignf(q0, a);
  b = copysignf(q1, b);
}
// 8 values divided by d (see divide_exact for `safe`)
__device__ __forceinline__ void divide_exact8(float (&v)[8], float d, float r, bool safe) {
  if (safe) {
    const uint64_t nd2 = f2_pack(-d, -d), r2 = f2_pack(r, r);
#pragma unroll
    for (int i = 0; i < 8; i += 2) divide_exact_pair(v[i], v[i + 1], nd2, r2);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __fdiv_rn(v[i], d);
  }
}

__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {  // low byte <- lo
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t cvt_e5m2x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// 8 floats -> 8 E2M1 codes in 4 bytes; element 2i goes to the HIGH nibble of byte i.
__device__ __forceinline__ uint32_t cvt_e2m1x8(const float (&v)[8]) {
  uint32_t r;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %1, %2;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %3, %4;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %5, %6;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %7, %8;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
      : "=r"(r)
      : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
  return r;
}
__device__ __forceinline__ float e4m3_to_f32(uint32_t code) {
  uint32_t h2;
  uint16_t c = static_cast<uint16_t>(code & 0xFF);
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(c));
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xFFFF)));
}
__device__ __forceinline__ float e5m2_to_f32(uint32_t code) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>((code & 0xFF) << 8)));
}
__device__ __forceinline__ float e2m1_to_f32(uint32_t code) {
  const float mag = (code & 4) ? ((code & 2) ? ((code & 1) ? 6.f : 4.f) : ((code & 1) ? 3.f : 2.f))
                               : ((code & 2) ? ((code & 1) ? 1.5f : 1.f) : ((code & 1) ? .5f : 0.f));
  return (code & 8) ? -mag : mag;
}

__device__ __forceinline__ float amax8(const float (&v)[8]) {
  float m = fabsf(v[0]);
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, fabsf(v[i]));
  return m;
}

__device__ __forceinline__ size_t sf_offset(int64_t row, int64_t kcol, int64_t ks_padded, bool swizzled,
                                            int64_t ks) {
  if (!swizzled) return static_cast<size_t>(row * ks + kcol);
  const int64_t mb = row >> 7, r = row & 127;
  return static_cast<size_t>(((mb * (ks_padded >> 2) + (kcol >> 2)) * 32 + (r & 31)) * 16 + (r >> 5) * 4 + (kcol & 3));
}


// One NVFP4 block: 16 values (two groups of 8) -> 8 bytes of E2M1 pairs and the E4M3 scale code.
//   s = e4m3(min(amax / d0, 448)) with d0 = max(6 * ts, 1e-12) and r0 = 1 / d0 correctly rounded;
//   q = e2m1(x / max(ts * f32(s), eps)).
__device__ __forceinline__ uint2 nvfp4_encode16(float (&v)[2][8], float ts, float d0, float r0, float eps, uint32_t& code) {
  const float m = fmaxf(amax8(v[0]), amax8(v[1]));
  const float s32 = fminf(divide_exact(m, d0, r0, (m * r0 < 1e30f) && (d0 > 1e-30f) && (d0 < 1e30f) && (m > 1e-30f)), 448.f);
  code = cvt_e4m3x2(s32, 0.f) & 0xFFu;
  const float d1 = fmaxf(__fmul_rn(ts, e4m3_to_f32(code)), eps);
  const float r = __frcp_rn(d1);
  // |x| <= m, so every quotient is below m * r * (1 + 2^-22); keep far from overflow, and
  // keep d1 / r in the normal range so the residuals are exact
  const bool safe = (m * r < 1e30f) && (d1 > 1e-30f) && (d1 < 1e30f);
  divide_exact8(v[0], d1, r, safe);
  divide_exact8(v[1], d1, r, safe);
  return make_uint2(cvt_e2m1x8(v[0]), cvt_e2m1x8(v[1]));
}

}  // namespace gnk
