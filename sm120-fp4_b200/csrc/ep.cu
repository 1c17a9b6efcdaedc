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

// ---------------------------------------------------------------------------------------------------------------------
// Variable-size exchange (prefill batches): a token row travels once to every rank that owns at least one of its experts.
namespace b200 {

constexpr int kEpMaxWorld = 16;

// One block. Thread i owns the contiguous tokens [i*c, (i+1)*c): per destination, an exclusive scan over the threads gives
// every sent (token, destination) its row in the send buffer - destination-major, token order within a destination.
// counts[d] rows go to rank d, offsets[d] is the first of them (offsets[world] = total), pos[t*world + d] the row of token
// t for destination d or -1, send_tok[row] = t.
__global__ void __launch_bounds__(1024) k_ep_plan(const int* __restrict__ ids, int m, int k, int world, int per, int* __restrict__ counts,
                                                  int* __restrict__ offsets, int* __restrict__ pos, int* __restrict__ send_tok) {
  __shared__ int wsum[32];
  __shared__ int s_off[kEpMaxWorld + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = (m + 1023) / 1024;
  const int t0 = tid * c, t1 = min(m, t0 + c);
  // pass 1: rows per destination
  int running = 0;
  for (int d = 0; d < world; ++d) {
    int mine = 0;
    for (int t = t0; t < t1; ++t) {
      bool hit = false;
      for (int j = 0; j < k; ++j) { const int e = ids[t * k + j]; hit |= e >= 0 && e / per == d; }
      mine += hit;
    }
    int inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int a = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += a; }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    int base = inc - mine;
    for (int w2 = 0; w2 < warp; ++w2) base += wsum[w2];
    int total = 0;
    for (int w2 = 0; w2 < 32; ++w2) total += wsum[w2];
    if (tid == 0) { s_off[d] = running; counts[d] = total; offsets[d] = running; }
    // pass 2 for this destination: rows of this thread's tokens
    int r = running + base;
    for (int t = t0; t < t1; ++t) {
      bool hit = false;
      for (int j = 0; j < k; ++j) { const int e = ids[t * k + j]; hit |= e >= 0 && e / per == d; }
      pos[t * world + d] = hit ? r : -1;
      if (hit) { send_tok[r] = t; ++r; }
    }
    running += total;
    __syncthreads();
  }
  if (tid == 0) offsets[world] = running;
}

// Block r (< offsets[world]): row r of the send buffer = token send_tok[r] for the destination whose range holds r.
__global__ void __launch_bounds__(128) k_ep_gather(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, const float* __restrict__ wts,
                                                   const int* __restrict__ send_tok, const int* __restrict__ offsets, int h, int k, int world,
                                                   int per, __nv_bfloat16* __restrict__ sx, int* __restrict__ meta) {
  for (int r = blockIdx.x; r < offsets[world]; r += gridDim.x) {
    int d = 0;
    while (d + 1 < world && r >= offsets[d + 1]) ++d;
    const int t = send_tok[r];
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * h);
    uint4* dst = reinterpret_cast<uint4*>(sx + (long long)r * h);
    for (int i = threadIdx.x; i < h / 8; i += blockDim.x) dst[i] = src[i];
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
      const int e = ids[t * k + j];
      const bool own = e >= 0 && e / per == d;
      meta[(long long)r * 2 * k + j] = own ? e - d * per : -1;
      meta[(long long)r * 2 * k + k + j] = __float_as_int(own ? wts[t * k + j] : 0.f);
    }
  }
}

// out[t] = bf16( sum over destinations d = 0..world-1, in that order, of float(back[pos[t, d]]) where pos >= 0 )
__global__ void __launch_bounds__(256) k_ep_combine_rows(const __nv_bfloat16* __restrict__ back, const int* __restrict__ pos, int m, int h, int world,
                                                         __nv_bfloat16* __restrict__ out) {
  const int chunks = h / 8;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < m * chunks; i += gridDim.x * blockDim.x) {
    const int t = i / chunks, c = i - t * chunks;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int d = 0; d < world; ++d) {
      const int r = pos[t * world + d];
      if (r < 0) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(back + (long long)r * h + c * 8);
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

// ids int32 [m, k] (global ids, negative = empty slot) -> counts int32 [world], offsets int32 [world + 1], pos int32
// [m, world], send_tok int32 [m * min(world, k)] (device buffers). 0 <= m <= 8192 * 8, world <= 16.
extern "C" int b200moe_ep_plan(const int* ids, int m, int k, int world, int experts_per_rank, int* counts, int* offsets, int* pos,
                               int* send_tok, void* stream) {
  if (!counts || !offsets || (m > 0 && (!ids || !pos || !send_tok))) return B200MOE_ERR_ARG;
  if (m < 0 || k < 1 || world < 1 || world > kEpMaxWorld || experts_per_rank < 1) return B200MOE_ERR_SHAPE;
  if (m == 0) {   // a rank with an empty batch still takes part in the exchange: it sends nothing to anybody
    B200_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int) * world, (cudaStream_t)stream));
    B200_CUDA_TRY(cudaMemsetAsync(offsets, 0, sizeof(int) * (world + 1), (cudaStream_t)stream));
    return B200MOE_OK;
  }
  k_ep_plan<<<1, 1024, 0, (cudaStream_t)stream>>>(ids, m, k, world, experts_per_rank, counts, offsets, pos, send_tok);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// rows [0, offsets[world]) of sx bf16 [rows, h] and meta int32 [rows, 2k] (local ids, then the weights' float bits)
extern "C" int b200moe_ep_gather(const void* x, const int* ids, const float* wts, const int* send_tok, const int* offsets, int h, int k, int world,
                                 int experts_per_rank, int max_rows, void* sx, int* meta, void* stream) {
  if (!x || !ids || !wts || !send_tok || !offsets || !sx || !meta) return B200MOE_ERR_ARG;
  if (h <= 0 || h % 8 || k < 1 || world < 1 || world > kEpMaxWorld || max_rows < 0) return B200MOE_ERR_SHAPE;
  if (max_rows == 0) return B200MOE_OK;
  const int grid = max_rows < 148 * 16 ? max_rows : 148 * 16;
  k_ep_gather<<<grid, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ids, wts, send_tok, offsets, h, k, world, experts_per_rank,
                                                      (__nv_bfloat16*)sx, meta);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// back bf16 [rows, h] (the partial rows in send-buffer order), pos int32 [m, world] -> out bf16 [m, h]
extern "C" int b200moe_ep_combine_rows(const void* back, const int* pos, int m, int h, int world, void* out, void* stream) {
  if (m > 0 && (!back || !pos || !out)) return B200MOE_ERR_ARG;
  if (m < 0 || h <= 0 || h % 8 || world < 1 || world > kEpMaxWorld) return B200MOE_ERR_SHAPE;
  if (m == 0) return B200MOE_OK;
  const int total = m * (h / 8);
  int grid = (total + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  k_ep_combine_rows<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)back, pos, m, h, world, (__nv_bfloat16*)out);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}
