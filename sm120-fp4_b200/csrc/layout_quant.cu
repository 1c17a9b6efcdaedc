// 128x4 block-scale swizzle and the bf16/fp32 -> NVFP4 quantizer, bit-exact restatements on the GPU of
// sm120fp4/layouts.py:39-78 and sm120fp4/reference.py:28-90. Both are byte-moving, HBM-bound kernels.
#include "common.cuh"
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include "nvfp4_math.cuh"

namespace b200 {

// ------------------------------------------------------------------------------------------------ 128x4 layout
// offset(r, c) = ((r/128) * nkt + c/4) * 512 + (r%32)*16 + ((r%128)/32)*4 + c%4, nkt = ceil(cols/4)
__device__ __forceinline__ long long sf_offset_128x4(int r, int c, int nkt) {
  return ((long long)(r >> 7) * nkt + (c >> 2)) * 512 + (r & 31) * 16 + ((r & 127) >> 5) * 4 + (c & 3);
}

// One thread per 4-byte group of the swizzled buffer (one row, four scale columns). Padding groups are written as zero.
__global__ void __launch_bounds__(256) k_to_128x4(const uint8_t* __restrict__ lin, uint8_t* __restrict__ swz, int batch,
                                                  int rows, int cols, int prow, int nkt) {
  const long long per = (long long)prow * nkt;
  const long long total = per * batch;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / per);
    const long long j = i % per;
    const int kt = (int)(j % nkt);
    const int r = (int)(j / nkt);
    uint32_t v = 0;
    if (r < rows) {
      const uint8_t* src = lin + ((long long)b * rows + r) * cols + kt * 4;
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (kt * 4 + c < cols) v |= (uint32_t)src[c] << (8 * c);
    }
    *reinterpret_cast<uint32_t*>(swz + (long long)b * prow * nkt * 4 + sf_offset_128x4(r, kt * 4, nkt)) = v;
  }
}

__global__ void __launch_bounds__(256) k_from_128x4(const uint8_t* __restrict__ swz, uint8_t* __restrict__ lin, int batch,
                                                    int rows, int cols, int prow, int nkt) {
  const long long per = (long long)rows * cols;
  const long long total = per * batch;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i / per);
    const long long j = i % per;
    const int c = (int)(j % cols);
    const int r = (int)(j / cols);
    lin[i] = swz[(long long)b * prow * nkt * 4 + sf_offset_128x4(r, c, nkt)];
  }
}

// ------------------------------------------------------------------------------------------------ quantizer
// amax over a flat array; non-negative floats order like their bit patterns, so one atomicMax per block suffices.
template <typename T>
__global__ void __launch_bounds__(256) k_amax(const T* __restrict__ x, long long n, unsigned* __restrict__ amax_bits) {
  float m = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf((float)x[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float wm[8];
  if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, wm[w]);
    atomicMax(amax_bits, __float_as_uint(m));
  }
}

// global_scale = reciprocal(max(amax, 1e-12)) * 2688: PyTorch evaluates the reference's `2688.0 / amax` with a Python
// scalar numerator as reciprocal-then-multiply (two roundings), and the golden vectors pin that.
__global__ void k_global_scale(const unsigned* __restrict__ amax_bits, float* __restrict__ gs) {
  const float amax = fmaxf(__uint_as_float(*amax_bits), 1e-12f);
  *gs = __fmul_rn(__frcp_rn(amax), 2688.0f);
}

// One thread per 16-element block. Destination row r reads source row src_row[r] (or r when src_row is null); a
// negative source row writes zero codes and zero scales (padding rows of a per-expert segment).
// sf_layout 0: row-major [rows, K/16]; 1: 128x4 swizzle over [rows, K/16] (rows padded by the caller's buffer).
template <typename T>
__global__ void __launch_bounds__(256) k_quantize_nvfp4(const T* __restrict__ x, const int* __restrict__ src_row, int rows,
                                                        int K, const float* __restrict__ gs_ptr, int gs_rows,
                                                        uint8_t* __restrict__ packed, uint8_t* __restrict__ sf, int sf_layout) {
  const int bpr = K >> 4;
  const int nkt = (bpr + 3) >> 2;
  const long long total = (long long)rows * bpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / bpr), b = (int)(i % bpr);
    const int s = src_row ? src_row[r] : r;
    uint2 pk = make_uint2(0u, 0u);
    uint8_t sb = 0;
    if (s >= 0) {
      float v[16];
      load16(x + (long long)s * K + b * 16, v);
      sb = quantize_block16(v, gs_ptr[gs_rows > 0 ? r / gs_rows : 0], pk);   // one global scale per gs_rows destination rows
    }
    *reinterpret_cast<uint2*>(packed + (long long)r * (K >> 1) + b * 8) = pk;
    if (sf_layout == 0) sf[(long long)r * bpr + b] = sb;
    else sf[sf_offset_128x4(r, b, nkt)] = sb;
  }
}

static inline int grid_for(long long work, int block, int cap = 148 * 16) {
  long long g = (work + block - 1) / block;
  if (g < 1) g = 1;
  return (int)(g > cap ? cap : g);
}

}  // namespace b200

using namespace b200;

extern "C" int b200moe_to_128x4(const void* sf_linear, void* sf_swizzled, int batch, int rows, int cols, void* stream) {
  if (!sf_linear || !sf_swizzled || batch < 0 || rows < 0 || cols < 0) return B200MOE_ERR_ARG;
  if (batch == 0 || rows == 0 || cols == 0) return B200MOE_OK;
  const int prow = (rows + 127) / 128 * 128, nkt = (cols + 3) / 4;
  k_to_128x4<<<grid_for((long long)batch * prow * nkt, 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)sf_linear, (uint8_t*)sf_swizzled, batch, rows, cols, prow, nkt);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

extern "C" int b200moe_from_128x4(const void* sf_swizzled, void* sf_linear, int batch, int rows, int cols, void* stream) {
  if (!sf_linear || !sf_swizzled || batch < 0 || rows < 0 || cols < 0) return B200MOE_ERR_ARG;
  if (batch == 0 || rows == 0 || cols == 0) return B200MOE_OK;
  const int prow = (rows + 127) / 128 * 128, nkt = (cols + 3) / 4;
  k_from_128x4<<<grid_for((long long)batch * rows * cols, 256), 256, 0, (cudaStream_t)stream>>>(
      (const uint8_t*)sf_swizzled, (uint8_t*)sf_linear, batch, rows, cols, prow, nkt);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// One global scale per group of `group_elems` consecutive elements: grid.y = group.
template <typename T>
__global__ void __launch_bounds__(256) k_amax_grouped(const T* __restrict__ x, long long group_elems, unsigned* __restrict__ amax_bits) {
  const T* xg = x + (long long)blockIdx.y * group_elems;
  float m = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < group_elems; i += (long long)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf((float)xg[i]));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float wm[8];
  if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, wm[w]);
    atomicMax(amax_bits + blockIdx.y, __float_as_uint(m));
  }
}
__global__ void k_global_scale_grouped(const unsigned* __restrict__ amax_bits, float* __restrict__ gs, int groups) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;
  if (g < groups) gs[g] = __fmul_rn(__frcp_rn(fmaxf(__uint_as_float(amax_bits[g]), 1e-12f)), 2688.0f);
}

extern "C" int b200moe_global_scale_grouped(const void* x, int dtype, int groups, long long group_elems, void* amax_scratch_u32,
                                            float* gs_out, void* stream) {
  if (!x || !amax_scratch_u32 || !gs_out || groups <= 0 || groups > 65535 || group_elems <= 0) return B200MOE_ERR_ARG;
  if (dtype != 0 && dtype != 1) return B200MOE_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  B200_CUDA_TRY(cudaMemsetAsync(amax_scratch_u32, 0, sizeof(unsigned) * groups, st));
  dim3 grid(grid_for(group_elems, 256 * 8, 64), groups);
  if (dtype == 0) k_amax_grouped<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, group_elems, (unsigned*)amax_scratch_u32);
  else k_amax_grouped<<<grid, 256, 0, st>>>((const float*)x, group_elems, (unsigned*)amax_scratch_u32);
  B200_LAUNCH_CHECK();
  k_global_scale_grouped<<<(groups + 127) / 128, 128, 0, st>>>((const unsigned*)amax_scratch_u32, gs_out, groups);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

extern "C" int b200moe_global_scale(const void* x, int dtype, long long n, void* amax_scratch_u32, float* gs_out, void* stream) {
  if (!x || !amax_scratch_u32 || !gs_out || n < 0) return B200MOE_ERR_ARG;
  if (dtype != 0 && dtype != 1) return B200MOE_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  B200_CUDA_TRY(cudaMemsetAsync(amax_scratch_u32, 0, sizeof(unsigned), st));
  if (n > 0) {
    if (dtype == 0) k_amax<<<grid_for(n, 256 * 8), 256, 0, st>>>((const __nv_bfloat16*)x, n, (unsigned*)amax_scratch_u32);
    else k_amax<<<grid_for(n, 256 * 8), 256, 0, st>>>((const float*)x, n, (unsigned*)amax_scratch_u32);
    B200_LAUNCH_CHECK();
  }
  k_global_scale<<<1, 1, 0, st>>>((const unsigned*)amax_scratch_u32, gs_out);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

extern "C" int b200moe_quantize_nvfp4(const void* x, int dtype, const int* src_row, int rows, int K, const float* global_scale,
                                      int gs_rows, void* packed, void* sf, int sf_layout, void* stream) {
  if (!x || !global_scale || !packed || !sf || rows < 0 || gs_rows < 0) return B200MOE_ERR_ARG;
  if (K <= 0 || K % 16) return B200MOE_ERR_SHAPE;
  if ((dtype != 0 && dtype != 1) || (sf_layout != 0 && sf_layout != 1)) return B200MOE_ERR_ARG;
  if (((uintptr_t)x & 15) || ((uintptr_t)packed & 7)) return B200MOE_ERR_ARG;
  if (rows == 0) return B200MOE_OK;
  cudaStream_t st = (cudaStream_t)stream;
  const int g = grid_for((long long)rows * (K / 16), 256);
  if (dtype == 0)
    k_quantize_nvfp4<<<g, 256, 0, st>>>((const __nv_bfloat16*)x, src_row, rows, K, global_scale, gs_rows, (uint8_t*)packed, (uint8_t*)sf, sf_layout);
  else
    k_quantize_nvfp4<<<g, 256, 0, st>>>((const float*)x, src_row, rows, K, global_scale, gs_rows, (uint8_t*)packed, (uint8_t*)sf, sf_layout);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}
