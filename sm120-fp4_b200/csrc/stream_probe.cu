// HBM streaming floor of the access patterns the MoE kernels use (the counterpart of the reference's k_stream probe,
// sm120fp4/kernels/micro_floor.py:59-95): every CTA pulls its share of a buffer through a shared-memory ring with TMA and
// does no math. Pattern 0: 2-D tensor boxes of 128 bytes x `box_rows` rows from a row-major [rows, pitch] matrix, K boxes
// of a row block visited in order (how weight tiles are read from the checkpoint layout). Pattern 1: contiguous chunks
// of `tile_bytes` with 1-D bulk copies (a tile-contiguous re-layout).
#include "common.cuh"
#include "ptx.cuh"
#include <cudaTypedefs.h>

namespace b200 {

struct StreamParams {
  CUtensorMap tm;
  const uint8_t* base;
  long long total_tiles;
  int pattern, box_rows, kboxes, tile_bytes, NS, producers;
  int* status;
};

__global__ void __launch_bounds__(192, 1) k_stream_probe(const __grid_constant__ StreamParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full[16], empty[16];
  __shared__ volatile int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NS = P.NS;
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  const long long t0 = (P.total_tiles * blockIdx.x) / gridDim.x, t1 = (P.total_tiles * (blockIdx.x + 1)) / gridDim.x;
  const int n = (int)(t1 - t0);
  const int slot_bytes = (P.tile_bytes + 1023) & ~1023;
  if (warp >= 1 && warp - 1 < P.producers) {
    if (lane == 0) {
      const int pw = warp - 1;
      for (int j = pw; j < n; j += P.producers) {
        const int slot = j % NS, use = j / NS;
        if (use >= 1 && !mbar_wait(&empty[slot], (use - 1) & 1, &abort_flag)) *P.status = 2;
        uint8_t* dst = smem + slot * slot_bytes;
        const long long t = t0 + j;
        mbar_expect_tx(&full[slot], P.tile_bytes);
        if (P.pattern == 0) {
          const long long rb = t / P.kboxes;
          const int kb = (int)(t % P.kboxes);
          tma_load_2d(dst, &P.tm, 128 * kb, (int)(rb * P.box_rows), &full[slot]);
        } else {
          bulk_load(dst, P.base + t * P.tile_bytes, P.tile_bytes, &full[slot]);
        }
      }
    }
  } else if (warp == 0) {
    if (lane == 0) {
      for (int j = 0; j < n; ++j) {
        const int slot = j % NS, use = j / NS;
        if (!mbar_wait(&full[slot], use & 1, &abort_flag)) *P.status = 1;
        mbar_arrive(&empty[slot]);
      }
    }
  }
  __syncthreads();
}

}  // namespace b200

using namespace b200;

// Stream `bytes` of `buf` once. pattern 0: buf is a row-major u8 matrix with `pitch` bytes per row, read as 128-byte x
// box_rows boxes; pattern 1: contiguous tiles of tile_bytes. Returns 0; time it with events around the call.
extern "C" int b200moe_stream_probe(const void* buf, long long bytes, int pattern, int pitch, int box_rows, int tile_bytes, int stages,
                                    int producers, int* status_dev, void* stream) {
  if (!buf || !status_dev || bytes <= 0 || stages < 2 || stages > 16 || producers < 1 || producers > 4) return B200MOE_ERR_ARG;
  StreamParams p;
  memset(&p, 0, sizeof(p));
  p.base = (const uint8_t*)buf;
  p.pattern = pattern, p.NS = stages, p.producers = producers, p.status = status_dev;
  if (pattern == 0) {
    if (pitch < 128 || pitch % 128 || box_rows < 8 || box_rows > 256) return B200MOE_ERR_ARG;
    const long long rows = bytes / pitch;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) return B200MOE_ERR_DEVICE;
    cuuint64_t dims[2] = {(cuuint64_t)pitch, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)pitch};
    cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1u, 1u};
    if (((PFN_cuTensorMapEncodeTiled_v12000)fn)(&p.tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(buf), dims, strides, box, estr,
                                                 CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                 CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return B200MOE_ERR_CUDA;
    p.box_rows = box_rows, p.kboxes = pitch / 128, p.tile_bytes = 128 * box_rows;
    p.total_tiles = (rows / box_rows) * p.kboxes;
  } else {
    if (tile_bytes < 1024 || tile_bytes % 16 || tile_bytes > 65536) return B200MOE_ERR_ARG;
    p.tile_bytes = tile_bytes;
    p.total_tiles = bytes / tile_bytes;
  }
  const int slot_bytes = (p.tile_bytes + 1023) & ~1023;
  const int smem = 1024 + stages * slot_bytes;
  if (smem > 227 * 1024) return B200MOE_ERR_LIMIT;
  int dev = 0, sms = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  B200_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  B200_CUDA_TRY(cudaFuncSetAttribute(k_stream_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  k_stream_probe<<<sms, 192, smem, (cudaStream_t)stream>>>(p);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}
