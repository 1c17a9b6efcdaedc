// W4A4 prefill MoE (many tokens): a ragged grouped GEMM on tcgen05.mma kind::mxf4nvf4 with TMEM accumulators. It replaces
// the third-party CUTLASS hand-off of the reference (sm120fp4/vllm_backend.py:123-168) with its own kernels and implements
// the reference's own W4A4 arithmetic (sm120fp4/kernels/bench_moe_baseline.py:53-74 with act_quant=True): x and the
// SiLU*mul activations quantised to NVFP4 by the bit-exact quantiser, fp32 accumulation, weighted sum over the top-k.
//
// Pipeline (all on the caller's stream, no host synchronisation):
//   route (route.cu) -> k_prefill_plan: per-expert row segments padded to 128-row tiles, gather map
//   k_quantize_records: bf16 x -> NVFP4 "tile records" (128 rows x 256 codes in the 128-byte-swizzle shared-memory image
//                       + four 512 B scale tiles, 18 KB contiguous), rows gathered per expert
//   k_prefill_gemm<1>:  FC1 tiles (128 rows x [64 up | 64 gate] columns), epilogue SiLU*mul + NVFP4 re-quantisation
//                       straight into FC2's tile records (scales written in the 128x4 order)
//   k_prefill_gemm<2>:  FC2 tiles (128 rows x 128 columns), epilogue alpha * routing weight -> bf16 rows per (token, expert)
//   k_prefill_combine:  out[token] = sum over its top-k rows, in slot order (deterministic)
// Both GEMM operands are streamed as 18 KB records with one bulk copy each (weights: the records built by
// b200moe_layer_prepack), so no tensor map is needed.
#include "common.cuh"
#include "tcgen05.cuh"
#include "nvfp4_math.cuh"
#include <string.h>

namespace b200 {

constexpr int kRec = 18432;          // one tile record: 16 KB codes image + 4 x 512 B scale tiles
constexpr int kPfStages = 5;         // ring stages of two records (A, B) each
constexpr int kPfThreads = 256;      // warps 0-3 epilogue, 4 MMA issuer, 5 scale copier, 6-7 TMA producers

// ------------------------------------------------------------------------------------------------ plan
// experts/offsets/pairs: the router's tables. Output: ntiles[0] = number of 128-row tiles, tile_expert[t], and for every
// padded row: src_tok (token index or -1) and row_pair (pair index or -1); dst_row[pair] = padded row of the pair.
__global__ void __launch_bounds__(1024) k_prefill_plan(const int* __restrict__ experts, const int* __restrict__ offsets,
                                                       const int* __restrict__ pairs, int Umax, int P, int top_k, int max_tiles,
                                                       int* __restrict__ ntiles, int* __restrict__ tile_expert, int* __restrict__ src_tok,
                                                       int* __restrict__ row_pair, int* __restrict__ dst_row) {
  extern __shared__ int sh[];   // tile_u[max_tiles], tile_first[max_tiles]
  int* tile_u = sh;
  int* tile_first = sh + max_tiles;
  __shared__ int s_nt;
  if (threadIdx.x == 0) {
    int nt = 0;
    for (int u = 0; u < Umax && experts[u] >= 0; ++u) {
      const int cnt = offsets[u + 1] - offsets[u];
      for (int j = 0; j * 128 < cnt && nt < max_tiles; ++j) {
        tile_u[nt] = u;
        tile_first[nt] = offsets[u] + j * 128;
        ++nt;
      }
    }
    s_nt = nt;
    ntiles[0] = nt;
  }
  __syncthreads();
  const int nt = s_nt;
  for (int t = threadIdx.x; t < nt; t += blockDim.x) tile_expert[t] = experts[tile_u[t]];
  for (int i = threadIdx.x; i < nt * 128; i += blockDim.x) {
    const int t = i >> 7, r = i & 127;
    const int u = tile_u[t];
    const int j = tile_first[t] + r;
    int tok = -1, pr = -1;
    if (j < offsets[u + 1]) {
      pr = pairs[j];
      tok = pr / top_k;
      dst_row[pr] = i;
    }
    src_tok[i] = tok;
    row_pair[i] = pr;
  }
}

// byte offset inside a tile record of 8 consecutive codes bytes (one 16-value block) of row r, K block b16 (0..15)
__device__ __forceinline__ int rec_code_offset(int r, int b16) { return r * 128 + ((((b16 >> 1) ^ (r & 7))) << 4) + (b16 & 1) * 8; }
__device__ __forceinline__ int rec_scale_offset(int r, int b16) { return 16384 + (b16 >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (b16 & 3); }

// ------------------------------------------------------------------------------------------------ x -> records
// One thread per 16-value block of a padded row. rec [ntiles][KB][18432]; K padded to KB*256 with zero codes/scales.
__global__ void __launch_bounds__(256) k_quantize_records(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src_tok,
                                                          const int* __restrict__ ntiles, int H, int KB, const float* __restrict__ gs_ptr,
                                                          uint8_t* __restrict__ rec) {
  const float gs = *gs_ptr;
  const long long total = (long long)ntiles[0] * 128 * KB * 16;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int b = (int)(i % (KB * 16));
    const long long row = i / (KB * 16);
    const int t = (int)(row >> 7), r = (int)(row & 127);
    const int tok = src_tok[row];
    uint2 pk = make_uint2(0u, 0u);
    uint8_t sb = 0;
    if (tok >= 0 && b * 16 < H) {
      float v[16];
      load16(x + (long long)tok * H + b * 16, v);
      sb = quantize_block16(v, gs, pk);
    }
    uint8_t* dst = rec + ((long long)t * KB + (b >> 4)) * kRec;
    *reinterpret_cast<uint2*>(dst + rec_code_offset(r, b & 15)) = pk;
    dst[rec_scale_offset(r, b & 15)] = sb;
  }
}

// ------------------------------------------------------------------------------------------------ grouped GEMM
struct PrefillParams {
  const uint8_t* arec;        // activation records [ntiles][KB][18432]
  const uint8_t* wrec;        // weight records [E][NBLK][KB][18432]
  const int* ntiles;
  const int* tile_expert;
  const int* row_pair;        // [ntiles*128] pair index or -1
  const float* alpha;         // per-expert weight scale
  const float* gs_in;         // global scale the A operand was quantised with
  const float* gs_out;        // PHASE 1: global scale for the activation re-quantisation
  const float* wts;           // PHASE 2: routing weights [P]
  uint8_t* orec;              // PHASE 1: FC2 activation records [ntiles][KB2][18432]
  __nv_bfloat16* y;           // PHASE 2: weighted rows [ntiles*128][H]
  int* status;
  int NBLK, KB, KT, KB2, H;
};

struct PfShared {
  uint64_t full[kPfStages], empty[kPfStages], sfr[kPfStages];
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

template <int PHASE>
__global__ void __launch_bounds__(kPfThreads, 1) k_prefill_gemm(const __grid_constant__ PrefillParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* ring = smem;   // kPfStages x [A record | B record], each record 1024-aligned (18432 = 18 * 1024)
  PfShared& S = *reinterpret_cast<PfShared*>(ring + kPfStages * 2 * kRec);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    for (int s = 0; s < kPfStages; ++s) { mbar_init(&S.full[s], 1); mbar_init(&S.empty[s], 1); mbar_init(&S.sfr[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&S.acc_full[b], 1); mbar_init(&S.acc_empty[b], 4); }
    S.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 4) { tmem_alloc(&S.tmem_base, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = S.tmem_base;
  const uint32_t tm_acc = tmem, tm_sfa = tmem + 256, tm_sfb = tmem + 256 + 16 * kPfStages;   // 2 x 128 | stages x 16 | stages x 16
  const int KB = P.KB, NBLK = P.NBLK;
  const long long nwork = (long long)P.ntiles[0] * NBLK;

  if (warp >= 6) {
    // ============================================================== producers: stage j of the CTA's sequence -> producer j mod 2
    if (lane == 0) {
      const int pw = warp - 6;
      long long j = 0;   // stage sequence number over all (work, kb) of this CTA
      for (long long w = blockIdx.x; w < nwork; w += gridDim.x) {
        const int t = (int)(w / NBLK), nblk = (int)(w % NBLK);
        const int e = P.tile_expert[t];
        for (int kb = 0; kb < KB; ++kb, ++j) {
          if ((j & 1) != pw) continue;
          const int slot = (int)(j % kPfStages);
          const long long use = j / kPfStages;
          if (use >= 1 && !mbar_wait(&S.empty[slot], (uint32_t)((use - 1) & 1), &S.abort_flag)) *P.status = 2;
          uint8_t* st = ring + slot * 2 * kRec;
          mbar_expect_tx(&S.full[slot], 2 * kRec);
          bulk_load(st, P.arec + ((long long)t * KB + kb) * kRec, kRec, &S.full[slot]);
          bulk_load(st + kRec, P.wrec + (((long long)e * NBLK + nblk) * KB + kb) * kRec, kRec, &S.full[slot]);
        }
      }
    }
    __syncwarp();
  } else if (warp == 4 || warp == 5) {
    // ============================================================== MMA issuer (4) and scale copier (5)
    if (lane == 0) {
      const bool copier = warp == 5;
      const uint32_t idesc = idesc_mxf4nvf4(128, 128);
      long long j = 0;
      int ab = 0, works = 0;
      uint32_t aph[2] = {0, 0};
      for (long long w = blockIdx.x; w < nwork; w += gridDim.x) {
        if (!copier) {
          if (works >= 2 && !mbar_wait(&S.acc_empty[ab], aph[ab] ^ 1u, &S.abort_flag)) *P.status = 5;
          tc_fence_after();
        }
        for (int kb = 0; kb < KB; ++kb, ++j) {
          const int slot = (int)(j % kPfStages);
          const uint32_t ph = (uint32_t)((j / kPfStages) & 1);
          const uint32_t sa = smem_u32(ring + slot * 2 * kRec), sb = sa + kRec;
          const int nkt = min(4, P.KT - 4 * kb);
          if (copier) {
            if (!mbar_wait(&S.full[slot], ph, &S.abort_flag)) *P.status = 1;
            tc_fence_after();
            for (int jj = 0; jj < nkt; ++jj) {
              tmem_cp_sf(tm_sfa + 16 * slot + 4 * jj, smem_desc_sf_tile(sa + 16384 + jj * 512));
              tmem_cp_sf(tm_sfb + 16 * slot + 4 * jj, smem_desc_sf_tile(sb + 16384 + jj * 512));
            }
            umma_commit(&S.sfr[slot]);
          } else {
            if (!mbar_wait(&S.sfr[slot], ph, &S.abort_flag)) *P.status = 8;
            if (!mbar_wait(&S.full[slot], ph, &S.abort_flag)) *P.status = 1;
            tc_fence_after();
            for (int jj = 0; jj < nkt; ++jj)
              umma_mxf4nvf4(tm_acc + 128 * ab, smem_desc_sw128_kmajor(sa) + 2 * jj, smem_desc_sw128_kmajor(sb) + 2 * jj, idesc,
                            tm_sfa + 16 * slot + 4 * jj, tm_sfb + 16 * slot + 4 * jj, (kb > 0 || jj > 0) ? 1u : 0u);
            umma_commit(&S.empty[slot]);
          }
        }
        if (!copier) {
          umma_commit(&S.acc_full[ab]);
          aph[ab] ^= 1u;
          ab ^= 1;
          ++works;
        }
      }
    }
    __syncwarp();
  } else {
    // ============================================================== epilogue: thread = accumulator row (token-expert pair)
    const int row = warp * 32 + lane;
    int ab = 0;
    uint32_t aph[2] = {0, 0};
    const float gs_in = *P.gs_in;
    for (long long w = blockIdx.x; w < nwork; w += gridDim.x) {
      const int t = (int)(w / NBLK), nblk = (int)(w % NBLK);
      const int e = P.tile_expert[t];
      if (!mbar_wait(&S.acc_full[ab], aph[ab], &S.abort_flag)) *P.status = 7;
      tc_fence_after();
      const uint32_t taddr = tm_acc + 128 * ab + ((uint32_t)(warp * 32) << 16);
      if (PHASE == 1) {
        // columns 0..63 = up, 64..127 = gate of intermediate columns 64*nblk..; SiLU*mul, re-quantise 4 blocks of 16
        const float s = P.alpha[e] / gs_in;
        const float gs_out = *P.gs_out;
        uint8_t* dst = P.orec + ((long long)t * P.KB2 + (nblk >> 2)) * kRec;
        uint32_t sfw = 0;
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
          uint32_t up[16], gt[16];
          tmem_ld_32x32b_x16(taddr + 16 * blk, up);
          tmem_ld_32x32b_x16(taddr + 64 + 16 * blk, gt);
          tmem_ld_wait();
          float a[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float g = __uint_as_float(gt[i]) * s, u = __uint_as_float(up[i]) * s;
            a[i] = g / (1.0f + __expf(-g)) * u;
          }
          uint2 pk;
          const uint8_t sb = quantize_block16(a, gs_out, pk);
          *reinterpret_cast<uint2*>(dst + rec_code_offset(row, 4 * (nblk & 3) + blk)) = pk;
          sfw |= (uint32_t)sb << (8 * blk);
        }
        *reinterpret_cast<uint32_t*>(dst + 16384 + (nblk & 3) * 512 + (row & 31) * 16 + (row >> 5) * 4) = sfw;
      } else {
        const int pr = P.row_pair[(long long)t * 128 + row];
        const float s = pr >= 0 ? P.alpha[e] / gs_in * P.wts[pr] : 0.f;
        __nv_bfloat16* yrow = P.y + ((long long)t * 128 + row) * P.H + 128 * nblk;
#pragma unroll
        for (int c0 = 0; c0 < 128; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(taddr + c0, r);
          tmem_ld_wait();
          if (pr >= 0) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * i]) * s, __uint_as_float(r[2 * i + 1]) * s);
              o[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(yrow + c0) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(yrow + c0 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&S.acc_empty[ab]);
      aph[ab] ^= 1u;
      ab ^= 1;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem, 512);
  if (S.abort_flag)
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
}

// ------------------------------------------------------------------------------------------------ combine
// out[tok, :] = sum_j y[dst_row[tok*k + j], :] in slot order, fp32 accumulation, one bf16 rounding.
__global__ void __launch_bounds__(256) k_prefill_combine(const __nv_bfloat16* __restrict__ y, const int* __restrict__ dst_row, int M, int top_k,
                                                         int H, __nv_bfloat16* __restrict__ out) {
  const int chunks = H / 8;
  const long long total = (long long)M * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int tok = (int)(i / chunks), c = (int)(i % chunks);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int r = dst_row[tok * top_k + j];
      if (r < 0) continue;   // empty slot
      const uint4 v = *reinterpret_cast<const uint4*>(y + (long long)r * H + c * 8);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += __uint_as_float(w[q] << 16);
        acc[2 * q + 1] += __uint_as_float(w[q] & 0xffff0000u);
      }
    }
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      o[q] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(out + (long long)tok * H + c * 8) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200moe_route(const int* ids, int P, int E, int Umax, int* experts, int* offsets, int* pairs, void* workspace,
                             long long workspace_bytes, void* stream);
extern "C" long long b200moe_route_workspace_bytes(int P, int E);

struct PrefillLayout {
  long long experts, offsets, pairs, route_ws, ntiles, tile_expert, src_tok, row_pair, dst_row, gs, status, xrec, arec, y, total;
  int max_tiles;
};

static inline long long pf_align(long long v) { return (v + 255) / 256 * 256; }

static PrefillLayout prefill_layout(int E, int H, int I, int top_k, int max_tokens) {
  PrefillLayout L;
  const long long P = (long long)max_tokens * top_k;
  const int KB1 = (H + 255) / 256, KB2 = (I + 255) / 256;
  L.max_tiles = (int)(P / 128 + E);
  long long o = 0;
  L.experts = o, o = pf_align(o + 4LL * E);
  L.offsets = o, o = pf_align(o + 4LL * (E + 1));
  L.pairs = o, o = pf_align(o + 4 * P);
  L.route_ws = o, o = pf_align(o + b200moe_route_workspace_bytes((int)P, E));
  L.ntiles = o, o += 256;
  L.tile_expert = o, o = pf_align(o + 4LL * L.max_tiles);
  L.src_tok = o, o = pf_align(o + 4LL * L.max_tiles * 128);
  L.row_pair = o, o = pf_align(o + 4LL * L.max_tiles * 128);
  L.dst_row = o, o = pf_align(o + 4 * P);
  L.gs = o, o += 256;
  L.status = o, o += 256;
  L.xrec = o, o = pf_align(o + (long long)L.max_tiles * KB1 * kRec);
  L.arec = o, o = pf_align(o + (long long)L.max_tiles * KB2 * kRec);
  L.y = o, o = pf_align(o + (long long)L.max_tiles * 128 * H * 2);
  L.total = o;
  return L;
}

long long b200_prefill_workspace_bytes(int E, int H, int I, int top_k, int max_tokens) {
  return prefill_layout(E, H, I, top_k, max_tokens).total;
}

__global__ void k_set2(float* p, float a, float b) { p[0] = a; p[1] = b; }

// w1t / w2t: the weight tile records of b200moe_layer_prepack. gs_x / gs_a: global scales of the two activation quantisations.
int b200_prefill_forward(int E, int H, int I, int top_k, const uint8_t* w1t, const uint8_t* w2t, const float* alpha1, const float* alpha2,
                         const void* x, const int* ids, const float* wts, int M, void* out, void* ws, long long ws_bytes, int ws_tokens,
                         float gs_x, float gs_a, int sms, cudaStream_t st) {
  const PrefillLayout L = prefill_layout(E, H, I, top_k, ws_tokens);
  if (ws_bytes < L.total || M > ws_tokens) return B200MOE_ERR_WORKSPACE;
  uint8_t* w = (uint8_t*)ws;
  const int P = M * top_k;
  const int Umax = E < P ? E : P;
  const int KB1 = (H + 255) / 256, KB2 = (I + 255) / 256, KT1 = (H / 16 + 3) / 4, KT2 = (I / 16 + 3) / 4;
  int* experts = (int*)(w + L.experts);
  int* offsets = (int*)(w + L.offsets);
  int* pairs = (int*)(w + L.pairs);
  int* ntiles = (int*)(w + L.ntiles);
  int* tile_expert = (int*)(w + L.tile_expert);
  int* src_tok = (int*)(w + L.src_tok);
  int* row_pair = (int*)(w + L.row_pair);
  int* dst_row = (int*)(w + L.dst_row);
  float* gs = (float*)(w + L.gs);
  int* status = (int*)(w + L.status);
  int rc = b200moe_route(ids, P, E, Umax, experts, offsets, pairs, w + L.route_ws, L.total - L.route_ws, st);
  if (rc != B200MOE_OK) return rc;
  B200_CUDA_TRY(cudaMemsetAsync(dst_row, 0xff, sizeof(int) * (size_t)P, st));
  const int max_tiles = P / 128 + Umax;
  k_prefill_plan<<<1, 1024, 2 * max_tiles * sizeof(int), st>>>(experts, offsets, pairs, Umax, P, top_k, max_tiles, ntiles, tile_expert, src_tok,
                                                                row_pair, dst_row);
  B200_LAUNCH_CHECK();
  k_set2<<<1, 1, 0, st>>>(gs, gs_x, gs_a);
  B200_LAUNCH_CHECK();
  k_quantize_records<<<sms * 8, 256, 0, st>>>((const __nv_bfloat16*)x, src_tok, ntiles, H, KB1, gs, w + L.xrec);
  B200_LAUNCH_CHECK();
  const int smem = 1024 + kPfStages * 2 * kRec + (int)sizeof(PfShared);
  static thread_local bool configured = false;
  if (!configured) {
    B200_CUDA_TRY(cudaFuncSetAttribute(k_prefill_gemm<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    B200_CUDA_TRY(cudaFuncSetAttribute(k_prefill_gemm<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = true;
  }
  PrefillParams p;
  memset(&p, 0, sizeof(p));
  p.ntiles = ntiles, p.tile_expert = tile_expert, p.row_pair = row_pair, p.status = status, p.H = H;
  // FC1
  p.arec = w + L.xrec, p.wrec = w1t, p.alpha = alpha1, p.gs_in = gs, p.gs_out = gs + 1, p.orec = w + L.arec;
  p.NBLK = I / 64, p.KB = KB1, p.KT = KT1, p.KB2 = KB2;
  k_prefill_gemm<1><<<sms, kPfThreads, smem, st>>>(p);
  B200_LAUNCH_CHECK();
  // FC2
  p.arec = w + L.arec, p.wrec = w2t, p.alpha = alpha2, p.gs_in = gs + 1, p.gs_out = nullptr, p.orec = nullptr;
  p.wts = wts, p.y = (__nv_bfloat16*)(w + L.y);
  p.NBLK = H / 128, p.KB = KB2, p.KT = KT2;
  k_prefill_gemm<2><<<sms, kPfThreads, smem, st>>>(p);
  B200_LAUNCH_CHECK();
  k_prefill_combine<<<sms * 8, 256, 0, st>>>((const __nv_bfloat16*)(w + L.y), dst_row, M, top_k, H, (__nv_bfloat16*)out);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

int b200_prefill_status_offset(int E, int H, int I, int top_k, int max_tokens, long long* off) {
  *off = prefill_layout(E, H, I, top_k, max_tokens).status;
  return 0;
}
