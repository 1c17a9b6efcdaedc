// W4A16 on an FP4 x FP4 tensor-core instruction: a 16-bit activation block is written as a short sum of NVFP4 blocks,
//     x = q1*s1/g1 + q2*s2/g2 + q3*s3/g3 + q4*s4/g4 + r,   g_t = g1 * 6^(t-1),   |r| <= blockmax(x) * 6^-4,
// each term the NVFP4 quantisation (E2M1 codes, E4M3 scale per 16 values) of the residual left by the terms before it.
// Shared by the decode kernel, its activation-expansion kernel and the W4A16 grouped GEMM of mid-sized batches.
#pragma once
#include "ptx.cuh"

namespace b200 {

constexpr int kTerms = 4;

__device__ __forceinline__ uint8_t tc_e4m3(float v) {   // RNE, saturating at 448, subnormals kept
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(v));
  return (uint8_t)(r & 0xff);
}
__device__ __forceinline__ float tc_e4m3_value(uint8_t b) {
  const uint32_t e = (b >> 3) & 15u, m = b & 7u;
  return e == 0 ? (float)m * 0.001953125f : __uint_as_float(((e + 120u) << 23) | (m << 20));
}

// 8 floats -> 8 E2M1 codes in one word (element 2j in the low nibble of byte j), hardware round-to-nearest-even,
// saturating. cvt.rn.satfinite.e2m1x2.f32 d, a, b puts a into the high and b into the low nibble of d.
__device__ __forceinline__ uint32_t cvt_f32x8_e2m1(const float* v) {
  uint32_t b[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    asm("{\n .reg .b8 t;\n cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n cvt.u32.u8 %0, t;\n}\n" : "=r"(b[i]) : "f"(v[2 * i + 1]), "f"(v[2 * i]));
  return (b[0] | (b[1] << 8)) | ((b[2] << 16) | (b[3] << 24));
}

// One 16-value block -> kTerms NVFP4 terms (residual expansion). g1: global scale of the first term; term t uses g1*6^t.
// codes[t] = 8 packed bytes (element 2j in the low nibble), sf[t] = E4M3 scale byte. The residual is taken against the
// codes and the scale actually emitted, so any rounding on the way (approximate reciprocal included) is absorbed by the
// next term.
// Returns true when the block's maximum lies beyond what the first term can hold (its scale clamps at 448, i.e. values
// above 2688 / g1): the later terms, with their larger global scales, cannot absorb the clipped part.
__device__ __forceinline__ bool expand_block16(float (&r)[16], float g1, uint2 (&codes)[kTerms], uint8_t (&sf)[kTerms]) {
  float g = g1, ginv = __frcp_rn(g1);
  bool clipped = false;
#pragma unroll
  for (int t = 0; t < kTerms; ++t) {
    float m[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = fmaxf(fabsf(r[i]), fabsf(r[i + 8]));
#pragma unroll
    for (int i = 0; i < 4; ++i) m[i] = fmaxf(m[i], m[i + 4]);
    const float amax = fmaxf(fmaxf(m[0], m[2]), fmaxf(m[1], m[3]));
    const float want = amax * (1.0f / 6.0f) * g;
    if (t == 0) clipped = want > 464.0f;   // 464 is the first value that no longer rounds down to 448
    const uint8_t sb = tc_e4m3(fminf(want, 448.0f));
    const float sv = tc_e4m3_value(sb);
    const float scale = sv > 0.f ? g * __frcp_rn(sv) : 0.f, back = sv * ginv;
    float sc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) sc[i] = r[i] * scale;
    const uint32_t lo = cvt_f32x8_e2m1(sc), hi = cvt_f32x8_e2m1(sc + 8);
    uint32_t dl[4], dh[4];
    cvt_e2m1x8_f16x2(lo, dl);
    cvt_e2m1x8_f16x2(hi, dh);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&dl[i]));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&dh[i]));
      r[2 * i] -= a.x * back;
      r[2 * i + 1] -= a.y * back;
      r[8 + 2 * i] -= b.x * back;
      r[8 + 2 * i + 1] -= b.y * back;
    }
    codes[t] = make_uint2(lo, hi);
    sf[t] = sb;
    g *= 6.0f;
    ginv *= (1.0f / 6.0f);
  }
  return clipped;
}

}  // namespace b200
