// Expert-parallel dispatch and combine for the fixed-capacity exchange (decode batches): two small kernels around the
// NCCL all-to-all, replacing a dozen framework element-wise launches. The reference has no expert parallelism (its
// `fits()` declines `use_ep`, sm120fp4/vllm_classes.py:46-47), so these entry points have no counterpart there.
#include "common.cuh"
#include <cuda_bf16.h>
#include <stdint.h>

namespace b200 {

// Block (row, dest): row `row` of the block sent to rank `dest` is token `row` (zeros beyond the batch), its top-k slots
// re-indexed to the destination's local experts; slots the destination does not own become id -1 / weight 0.
// meta[dest][row][0..k) = local ids (int32), meta[dest][row][k..2k) = routing weights (float bits).
__global__ void __launch_bounds__(128) k_ep_dispatch(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids,
                                                     const float* __restrict__ wts, int m, int h, int k, int per, int cap,
                                                     __nv_bfloat16* __restrict__ sx, int* __restrict__ meta) {
  const int row = blockIdx.x, dest = blockIdx.y;
  const long long o = (long long)dest * cap + row;
  uint4* dst = reinterpret_cast<uint4*>(sx + o * h);
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)row * h);
  for (int i = threadIdx.x; i < h / 8; i += blockDim.x) dst[i] = row < m ? src[i] : make_uint4(0u, 0u, 0u, 0u);
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    int id = -1;
    float w = 0.f;
    if (row < m) {
      const int e = ids[row * k + j];
      if (e >= 0 && e / per == dest) { id = e - dest * per; w = wts[row * k + j]; }
    }
    meta[o * 2 * k + j] = id;
    meta[o * 2 * k + k + j] = __float_as_int(w);
  }
}

// out[t] = bf16( sum over ranks r = 0..world-1, in that order, of float(y[r][t]) ): bit-identical from call to call.
__global__ void __launch_bounds__(256) k_ep_combine(const __nv_bfloat16* __restrict__ y, int m, int h, int world, int cap,
                                                    __nv_bfloat16* __restrict__ out) {
  const int chunks = h / 8;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < m * chunks; i += gridDim.x * blockDim.x) {
    const int t = i / chunks, c = i - t * chunks;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const uint4 v = *reinterpret_cast<const uint4*>(y + ((long long)r * cap + t) * h + c * 8);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += __uint_as_float(w4[q] << 16);
        acc[2 * q + 1] += __uint_as_float(w4[q] & 0xffff0000u);
      }
    }
    uint32_t o4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat162 hh = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      o4[q] = *reinterpret_cast<const uint32_t*>(&hh);
    }
    *reinterpret_cast<uint4*>(out + (long long)t * h + c * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
  }
}

}  // namespace b200

using namespace b200;

// x bf16 [m, h], ids int32 [m, k] (global expert ids, negative = empty slot), wts f32 [m, k] -> sx bf16 [world, cap, h],
// meta int32 [world, cap, 2k]. experts_per_rank = E / world; m <= cap; h a multiple of 8.
extern "C" int b200moe_ep_dispatch(const void* x, const int* ids, const float* wts, int m, int h, int k, int world, int experts_per_rank,
                                   int cap, void* sx, int* meta, void* stream) {
  if (!x || !ids || !wts || !sx || !meta) return B200MOE_ERR_ARG;
  if (m < 0 || m > cap || h <= 0 || h % 8 || k < 1 || world < 1 || experts_per_rank < 1 || cap < 1) return B200MOE_ERR_SHAPE;
  k_ep_dispatch<<<dim3(cap, world), 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ids, wts, m, h, k, experts_per_rank, cap,
                                                                     (__nv_bfloat16*)sx, meta);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// y bf16 [world, cap, h] (the partial rows that came back, block r from rank r) -> out bf16 [m, h]
extern "C" int b200moe_ep_combine(const void* y, int m, int h, int world, int cap, void* out, void* stream) {
  if (!y || !out) return B200MOE_ERR_ARG;
  if (m < 0 || m > cap || h <= 0 || h % 8 || world < 1) return B200MOE_ERR_SHAPE;
  if (m == 0) return B200MOE_OK;
  const int total = m * (h / 8);
  k_ep_combine<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)y, m, h, world, cap, (__nv_bfloat16*)out);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}
