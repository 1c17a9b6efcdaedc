// NVFP4 quantisation arithmetic in the exact operation order of sm120fp4/reference.py:28-90 (bit-exact with the reference's
// CPU code): block amax / 6 (IEEE division) * gs, clamp 448, E4M3 round-to-nearest-even; scale = gs / sf (IEEE division);
// E2M1 codes rounded to nearest with ties to the even code, saturating at 6, the sign bit kept on zero - which is exactly
// the hardware conversion cvt.rn.satfinite.e2m1x2.f32 (the threshold form below states the same rule in plain C).
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

// 8 floats -> 8 E2M1 codes in one word (element 2j in the low nibble of byte j). cvt.rn.satfinite.e2m1x2.f32 d, a, b puts
// a into the high and b into the low nibble of d.
__device__ __forceinline__ uint32_t e2m1x8_rn(const float* v) {
  uint32_t b[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    asm("{\n .reg .b8 t;\n cvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n cvt.u32.u8 %0, t;\n}\n" : "=r"(b[i]) : "f"(v[2 * i + 1]), "f"(v[2 * i]));
  return (b[0] | (b[1] << 8)) | ((b[2] << 16) | (b[3] << 24));
}

// Quantize one 16-element block: returns the E4M3 scale byte, writes 8 packed bytes.
__device__ __forceinline__ uint8_t quantize_block16(const float (&v)[16], float gs, uint2& packed) {
  float m[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) m[i] = fmaxf(fabsf(v[i]), fabsf(v[i + 8]));
#pragma unroll
  for (int i = 0; i < 4; ++i) m[i] = fmaxf(m[i], m[i + 4]);
  const float amax = fmaxf(fmaxf(m[0], m[2]), fmaxf(m[1], m[3]));
  const float sf_f = fminf(__fmul_rn(__fdiv_rn(amax, 6.0f), gs), 448.0f);
  const __nv_fp8_storage_t sfb = __nv_cvt_float_to_fp8(sf_f, __NV_SATFINITE, __NV_E4M3);  // RNE, subnormals kept
  const float sf_val = __half2float(__half(__nv_cvt_fp8_to_halfraw(sfb, __NV_E4M3)));
  const float scale = sf_val > 0.f ? __fdiv_rn(gs, sf_val) : 0.f;
  float sc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) sc[i] = __fmul_rn(v[i], scale);
  packed = make_uint2(e2m1x8_rn(sc), e2m1x8_rn(sc + 8));
  return (uint8_t)sfb;
}

// The same with the second division looked up: `table[b]` = gs / value(E4M3 byte b) for b = 0..127 (0 for b = 0), filled once
// per thread block by fill_scale_table with the very division the function above performs, so the results are identical.
__device__ __forceinline__ void fill_scale_table(float* table, float gs, int tid, int nthreads) {
  for (int b = tid; b < 128; b += nthreads) {
    const float sf_val = __half2float(__half(__nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3)));
    table[b] = sf_val > 0.f && sf_val == sf_val ? __fdiv_rn(gs, sf_val) : 0.f;
  }
}
__device__ __forceinline__ uint8_t quantize_block16_t(const float (&v)[16], float gs, const float* __restrict__ table, uint2& packed) {
  float m[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) m[i] = fmaxf(fabsf(v[i]), fabsf(v[i + 8]));
#pragma unroll
  for (int i = 0; i < 4; ++i) m[i] = fmaxf(m[i], m[i + 4]);
  const float amax = fmaxf(fmaxf(m[0], m[2]), fmaxf(m[1], m[3]));
  const float sf_f = fminf(__fmul_rn(__fdiv_rn(amax, 6.0f), gs), 448.0f);
  const __nv_fp8_storage_t sfb = __nv_cvt_float_to_fp8(sf_f, __NV_SATFINITE, __NV_E4M3);
  const float scale = table[sfb & 127];
  float sc[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) sc[i] = __fmul_rn(v[i], scale);
  packed = make_uint2(e2m1x8_rn(sc), e2m1x8_rn(sc + 8));
  return (uint8_t)sfb;
}

}  // namespace b200
