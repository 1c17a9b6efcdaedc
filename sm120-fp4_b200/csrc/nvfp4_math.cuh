// NVFP4 quantisation arithmetic in the exact operation order of sm120fp4/reference.py:28-90 (bit-exact with the reference's
// CPU code): block amax / 6 (IEEE division) * gs, clamp 448, E4M3 round-to-nearest-even; scale = gs / sf (IEEE division);
// E2M1 codes by thresholds with ties to the even code and the sign bit kept on zero.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

namespace b200 {

__device__ __forceinline__ uint32_t e2m1_code(float v) {
  // round to nearest, ties to the even code, saturate at 6, sign bit kept on zero (sm120fp4/reference.py:28-44)
  const float m = fabsf(v);
  uint32_t c = (m > 0.25f) + (m >= 0.75f) + (m > 1.25f) + (m >= 1.75f) + (m > 2.5f) + (m >= 3.5f) + (m > 5.0f);
  return c | ((__float_as_uint(v) >> 31) << 3);
}

__device__ __forceinline__ void load16(const __nv_bfloat16* p, float (&v)[16]) {
  const uint4 a = reinterpret_cast<const uint4*>(p)[0], b = reinterpret_cast<const uint4*>(p)[1];
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void load16(const float* p, float (&v)[16]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 f = reinterpret_cast<const float4*>(p)[i];
    v[4 * i] = f.x, v[4 * i + 1] = f.y, v[4 * i + 2] = f.z, v[4 * i + 3] = f.w;
  }
}

// Quantize one 16-element block: returns the E4M3 scale byte, writes 8 packed bytes.
__device__ __forceinline__ uint8_t quantize_block16(const float (&v)[16], float gs, uint2& packed) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(v[i]));
  const float sf_f = fminf(__fmul_rn(__fdiv_rn(amax, 6.0f), gs), 448.0f);
  const __nv_fp8_storage_t sfb = __nv_cvt_float_to_fp8(sf_f, __NV_SATFINITE, __NV_E4M3);  // RNE, subnormals kept
  const float sf_val = __half2float(__half(__nv_cvt_fp8_to_halfraw(sfb, __NV_E4M3)));
  const float scale = sf_val > 0.f ? __fdiv_rn(gs, sf_val) : 0.f;
  uint32_t lo = 0, hi = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) lo |= e2m1_code(__fmul_rn(v[i], scale)) << (4 * i);
#pragma unroll
  for (int i = 0; i < 8; ++i) hi |= e2m1_code(__fmul_rn(v[8 + i], scale)) << (4 * i);
  packed = make_uint2(lo, hi);
  return (uint8_t)sfb;
}

}  // namespace b200
