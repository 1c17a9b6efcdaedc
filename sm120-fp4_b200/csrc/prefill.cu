// W4A4 prefill MoE (many tokens): a ragged grouped GEMM on tcgen05.mma kind::mxf4nvf4 with TMEM accumulators. It replaces
// the third-party CUTLASS hand-off of the reference (sm120fp4/vllm_backend.py:123-168) with its own kernels and implements
// the reference's own W4A4 arithmetic (sm120fp4/kernels/bench_moe_baseline.py:53-74 with act_quant=True): x and the
// SiLU*mul activations quantised to NVFP4 by the bit-exact quantiser, fp32 accumulation, weighted sum over the top-k.
//
// Pipeline (all on the caller's stream, no host synchronisation):
//   route (route.cu) -> k_prefill_rowmap: per-expert row segments padded to 128-row tiles (the tile plan) and the map between
//                       token-expert pairs and operand rows
//   k_quantize_scatter: bf16 x -> NVFP4 "tile records" (128 rows x 256 codes in the 128-byte-swizzle shared-memory image
//                       + four 512 B scale tiles, 18 KB contiguous): every token row quantised once, stored to its pairs' rows
//   k_prefill_gemm<1>:  FC1 tiles (128 rows x [64 up | 64 gate] columns), epilogue SiLU*mul + NVFP4 re-quantisation
//                       straight into FC2's tile records (scales written in the 128x4 order)
//   k_prefill_gemm<2>:  FC2 tiles (128 rows x 128 columns), epilogue alpha * routing weight -> bf16 rows per (token, expert)
//   k_prefill_combine:  out[token] = sum over its top-k rows, in slot order (deterministic)
// Both GEMM operands are streamed as 18 KB records with one bulk copy each (weights: the records built by
// b200moe_layer_prepack), so no tensor map is needed.
#include "common.cuh"
#include "tcgen05.cuh"
#include "nvfp4_math.cuh"
#include "expand.cuh"
#include <string.h>
#include <stdlib.h>

namespace b200 {

constexpr int kRec = 18432;          // one tile record: 16 KB codes image + 4 x 512 B scale tiles
constexpr int kPfStages = 5;         // ring stages of two records (A, B) each
constexpr int kPfThreads = 256;      // warps 0-3 epilogue, 4 MMA issuer, 5 scale copier, 6-7 TMA producers
// W4A16 phases (3, 4): the operand tile holds 64 rows (16 token-expert pairs x four terms) in 10 KB records (8 KB codes
// image + four 512-byte scale tiles whose row groups 2 and 3 stay zero). The MMA still spans 128 rows: rows 64..127 read
// whatever follows the record in shared memory, with zero scales, and their accumulator rows are ignored. Half the
// resident bytes leave room for a weight ring twice as deep, which is what a batch that touches every expert once needs.
constexpr int kMidRec = 8192 + 2048;

// Ablation switches of the resident-operand GEMM (what a phase costs when a part of it is left out) exist only in a
// diagnostic build (-DB200_PF_ABLATE, read from B200MOE_PF_ABLATE at launch); the product build compiles them away.
#ifdef B200_PF_ABLATE
#define PF_ABLATE(bit) (P.dbg & (bit))
#else
#define PF_ABLATE(bit) false
#endif

// byte offset inside a tile record of 8 consecutive codes bytes (one 16-value block) of row r, K block b16 (0..15)
__device__ __forceinline__ int rec_code_offset(int r, int b16) { return r * 128 + ((((b16 >> 1) ^ (r & 7))) << 4) + (b16 & 1) * 8; }
__device__ __forceinline__ int rec_scale_offset(int r, int b16) { return 16384 + (b16 >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (b16 & 3); }

// ------------------------------------------------------------------------------------------------ row map
// The tile plan of the W4A4 path and the map between token-expert pairs and operand rows, in one launch. Every block
// repeats the (tiny) scan over the touched experts in shared memory: expert u owns tiles [tbase[u], tbase[u+1]) of 128
// rows; block 0 also writes the tile tables the GEMM kernels read. Then, grid-wide, one thread per padded operand row:
// row_pair[row] = the pair the row holds (-1 on the padding rows of an expert's last tile), dst_row[pair] = row; the
// scale bytes of padding rows are zeroed in the x records (a zero scale silences whatever codes the row holds, so their
// codes are never written). Pairs whose slot is empty (negative id) are not in `pairs`: they get dst_row = -1 here.
__global__ void __launch_bounds__(256) k_prefill_rowmap(const int* __restrict__ ids, int P, const int* __restrict__ experts,
                                                        const int* __restrict__ offsets, const int* __restrict__ pairs, int Umax, int max_tiles,
                                                        int KB, int even, int* __restrict__ ntiles, int* __restrict__ tile_expert,
                                                        int* __restrict__ tile_first, int* __restrict__ tile_end, uint8_t* __restrict__ rec,
                                                        int* __restrict__ row_pair, int* __restrict__ dst_row) {
  __shared__ int wsum[8];
  __shared__ int tbase[257];   // first tile of touched expert u; tbase[U..] = total
  __shared__ int s_lo[256], s_hi[256];
  const int u = threadIdx.x, lane = u & 31, warp = u >> 5;
  int e = -1, lo = 0, hi = 0;
  if (u < Umax) {
    e = experts[u];
    if (e >= 0) { lo = offsets[u]; hi = offsets[u + 1]; }
  }
  // `even`: an expert's tile count is rounded up to an even number (CTA pairs take two tiles of one expert at a time); the
  // extra tile holds padding rows only
  const int mine = even ? 2 * ((hi - lo + 255) >> 8) : (hi - lo + 127) >> 7;
  int inc = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += a;
  }
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  int base = inc - mine;
  for (int w2 = 0; w2 < warp; ++w2) base += wsum[w2];
  tbase[u] = base;
  s_lo[u] = lo, s_hi[u] = hi;
  if (u == 255) tbase[256] = base + mine;
  __syncthreads();
  const int NT = min(tbase[256], max_tiles);
  if (blockIdx.x == 0) {
    if (u == 0) ntiles[0] = NT;
    for (int j = 0; j < mine && base + j < max_tiles; ++j) {
      tile_expert[base + j] = e;
      tile_first[base + j] = lo + j * 128;
      tile_end[base + j] = hi;
    }
  }
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x, gsz = gridDim.x * blockDim.x;
  for (int p = gtid; p < P; p += gsz)
    if (ids[p] < 0) dst_row[p] = -1;
  for (int row = gtid; row < NT * 128; row += gsz) {
    const int t = row >> 7, r = row & 127;
    int a = 0, b = 255;   // the touched expert whose tile range holds t: last u with tbase[u] <= t
    while (a < b) {
      const int mid = (a + b + 1) >> 1;
      if (tbase[mid] <= t) a = mid; else b = mid - 1;
    }
    const int j = s_lo[a] + (t - tbase[a]) * 128 + r;
    const int pr = j < s_hi[a] ? pairs[j] : -1;
    row_pair[row] = pr;
    if (pr >= 0) {
      dst_row[pr] = row;
    } else {
      for (int kb = 0; kb < KB; ++kb) {
        uint8_t* sfp = rec + ((long long)t * KB + kb) * kRec + 16384 + (r & 31) * 16 + (r >> 5) * 4;
#pragma unroll
        for (int q = 0; q < 4; ++q) *reinterpret_cast<uint32_t*>(sfp + q * 512) = 0u;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ x -> records
// One block of 128 threads per token, one thread per 16-value block (a second round for rows of more than 2048 values):
// the token's row is read and quantised ONCE (the reference's block arithmetic, bit-exact) and its codes and scale bytes are
// then stored into the record rows of each of its top_k pairs (dst_row, -1 = empty slot). rec [ntiles][KB][18432]; blocks
// beyond H inside the last K box are written as zero codes and zero scales.
__global__ void __launch_bounds__(128) k_quantize_scatter(const __nv_bfloat16* __restrict__ x, const int* __restrict__ dst_row, int M, int H,
                                                          int KB, int top_k, float gs, uint8_t* __restrict__ rec) {
  __shared__ float s_scale[128];   // gs / (E4M3 value) for every scale byte: one division per table entry instead of one per block
  __shared__ int s_row[16];
  fill_scale_table(s_scale, gs, threadIdx.x, blockDim.x);
  const int tok = blockIdx.x;
  if (threadIdx.x < top_k) s_row[threadIdx.x] = dst_row[tok * top_k + threadIdx.x];
  __syncthreads();
  const int nblk = KB * 16;
  for (int b = threadIdx.x; b < ((nblk + 127) & ~127); b += 128) {   // whole warps stay in the loop: the shuffles below need them
    uint2 pk = make_uint2(0u, 0u);
    uint32_t sb = 0;
    if (b < nblk && b * 16 < H) {
      float v[16];
      load16(x + (long long)tok * H + b * 16, v);
      sb = quantize_block16_t(v, gs, s_scale, pk);
    }
    // the four scale bytes of one 64-value K step are adjacent in a record: lane 4i gathers them into one 32-bit store
    uint32_t sf4 = sb | (__shfl_down_sync(0xffffffffu, sb, 1) << 8);
    sf4 |= __shfl_down_sync(0xffffffffu, sf4, 2) << 16;
    const int kb = b >> 4, b16 = b & 15;
    if (b >= nblk) continue;
    for (int j = 0; j < top_k; ++j) {
      const int row = s_row[j];
      if (row < 0) continue;
      uint8_t* dst = rec + ((long long)(row >> 7) * KB + kb) * kRec;
      const int r = row & 127;
      *reinterpret_cast<uint2*>(dst + rec_code_offset(r, b16)) = pk;
      if ((b & 3) == 0) *reinterpret_cast<uint32_t*>(dst + rec_scale_offset(r, b16)) = sf4;
    }
  }
}

// ------------------------------------------------------------------------------------------------ x -> W4A16 records
// Mid-sized batches (17 tokens up to a few hundred) keep the decode path's W4A16 arithmetic but run as a grouped GEMM over
// per-expert gathered rows: a tile of 64 operand rows holds 16 token-expert pairs x four NVFP4 terms of the pair's token
// row (row 4p + t = term t of pair p), so that an expert's weight records are streamed once for all of its pairs. Two
// launches build the records (tile plan, pair-row map and the reset of the row table in one kernel; token amax and
// expansion in one token-major kernel that expands a token's row ONCE and stores it into the rows of each of its pairs) -
// a mid-sized batch is bound by launches, not by bytes.
//
// Row map: every block repeats the scan over the touched experts (tiles of 16 pairs); block 0 writes the tile tables. One
// thread per pair row of every tile: row_pair of its four term rows, dst_row of the pair; the scale bytes of pair rows
// that hold no pair are zeroed in the x records (so their codes never need writing).
__global__ void __launch_bounds__(256) k_mid_rowmap(const int* __restrict__ ids, int P, const int* __restrict__ experts, const int* __restrict__ offsets,
                                                    const int* __restrict__ pairs, int Umax, int max_tiles, int KB, int* __restrict__ ntiles,
                                                    int* __restrict__ tile_expert, int* __restrict__ tile_first, int* __restrict__ tile_end,
                                                    uint8_t* __restrict__ rec, int* __restrict__ row_pair, int* __restrict__ dst_row) {
  __shared__ int wsum[8];
  __shared__ int tbase[257];
  __shared__ int s_lo[256], s_hi[256];
  const int u = threadIdx.x, lane = u & 31, warp = u >> 5;
  int e = -1, lo = 0, hi = 0;
  if (u < Umax) {
    e = experts[u];
    if (e >= 0) { lo = offsets[u]; hi = offsets[u + 1]; }
  }
  const int mine = (hi - lo + 15) >> 4;
  int inc = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int a = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += a;
  }
  if (lane == 31) wsum[warp] = inc;
  __syncthreads();
  int base = inc - mine;
  for (int w2 = 0; w2 < warp; ++w2) base += wsum[w2];
  tbase[u] = base;
  s_lo[u] = lo, s_hi[u] = hi;
  if (u == 255) tbase[256] = base + mine;
  __syncthreads();
  const int NT = min(tbase[256], max_tiles);
  if (blockIdx.x == 0) {
    if (u == 0) ntiles[0] = NT;
    for (int j = 0; j < mine && base + j < max_tiles; ++j) {
      tile_expert[base + j] = e;
      tile_first[base + j] = lo + j * 16;
      tile_end[base + j] = hi;
    }
  }
  const int gtid = blockIdx.x * blockDim.x + threadIdx.x, gsz = gridDim.x * blockDim.x;
  for (int p = gtid; p < P; p += gsz)
    if (ids[p] < 0) dst_row[p] = -1;
  // one thread per (pair row, K box): the row's entry of the tables (by the thread of box 0) and, for a row that holds no
  // pair, the sixteen scale words of its four term rows in this box's record
  for (long long it = gtid; it < (long long)NT * 16 * KB; it += gsz) {
    const int prow = (int)(it / KB), kb = (int)(it - (long long)prow * KB);
    const int t = prow >> 4, p = prow & 15;
    int a = 0, b = 255;
    while (a < b) {
      const int mid = (a + b + 1) >> 1;
      if (tbase[mid] <= t) a = mid; else b = mid - 1;
    }
    const int j = s_lo[a] + (t - tbase[a]) * 16 + p;
    const int pr = j < s_hi[a] ? pairs[j] : -1;
    if (kb == 0) {
#pragma unroll
      for (int q = 0; q < kTerms; ++q) row_pair[t * 64 + 4 * p + q] = pr;
      if (pr >= 0) dst_row[pr] = prow;
    }
    if (pr < 0) {
#pragma unroll
      for (int q = 0; q < kTerms; ++q) {
        const int r = 4 * p + q;
        uint8_t* sfp = rec + ((long long)t * KB + kb) * kMidRec + 8192 + (r & 31) * 16 + (r >> 5) * 4;
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) *reinterpret_cast<uint32_t*>(sfp + jj * 512) = 0u;
      }
    }
  }
}

// One block of 128 threads per token: token amax, then every 16-value block expanded into four NVFP4 terms ONCE and stored
// into the four term rows of each of the token's pairs (dst_row[pair] = tile * 16 + pair row); the first four threads also
// write the rows' 1 / g_t.
__global__ void __launch_bounds__(128) k_expand_scatter(const __nv_bfloat16* __restrict__ x, const int* __restrict__ dst_row, int M, int H, int KB,
                                                        int top_k, uint8_t* __restrict__ rec, float* __restrict__ rowscale) {
  __shared__ float wm[4];
  __shared__ int s_row[16];
  const int tok = blockIdx.x, tid = threadIdx.x;
  if (tid < top_k) s_row[tid] = dst_row[tok * top_k + tid];
  float m = 0.f;
  for (int i = tid * 8; i < H; i += 128 * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(x + (long long)tok * H + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) m = fmaxf(m, fmaxf(fabsf(__uint_as_float(w[q] << 16)), fabsf(__uint_as_float(w[q] & 0xffff0000u))));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((tid & 31) == 0) wm[tid >> 5] = m;
  __syncthreads();
  m = fmaxf(fmaxf(wm[0], wm[1]), fmaxf(wm[2], wm[3]));
  const float g1 = 2688.0f / fmaxf(m, 1e-30f);
  if (tid < kTerms) {
    float g = g1;
    for (int q = 0; q < tid; ++q) g *= 6.0f;
    for (int j = 0; j < top_k; ++j) {
      const int prow = s_row[j];
      if (prow >= 0) rowscale[(prow >> 4) * 64 + 4 * (prow & 15) + tid] = 1.0f / g;
    }
  }
  const int nblk = KB * 16;
  for (int b = tid; b < nblk; b += 128) {
    uint2 codes[kTerms];
    uint8_t sf[kTerms];
    if (b * 16 < H) {
      float v[16];
      load16(x + (long long)tok * H + b * 16, v);
      expand_block16(v, g1, codes, sf);
    } else {
#pragma unroll
      for (int q = 0; q < kTerms; ++q) { codes[q] = make_uint2(0u, 0u); sf[q] = 0; }
    }
    for (int j = 0; j < top_k; ++j) {
      const int prow = s_row[j];
      if (prow < 0) continue;
      uint8_t* dst = rec + ((long long)(prow >> 4) * KB + (b >> 4)) * kMidRec;
      const int p = prow & 15;
#pragma unroll
      for (int q = 0; q < kTerms; ++q) {
        const int r = 4 * p + q;
        *reinterpret_cast<uint2*>(dst + rec_code_offset(r, b & 15)) = codes[q];
        dst[8192 + ((b & 15) >> 2) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (b & 3)] = sf[q];
      }
    }
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
  float gs_in;                // global scale the A operand was quantised with
  float gs_out;               // PHASE 1: global scale for the activation re-quantisation
  const float* wts;           // PHASE 2: routing weights [P]
  uint8_t* orec;              // PHASE 1: FC2 activation records [ntiles][KB2][18432]
  __nv_bfloat16* y;           // PHASE 2: weighted rows [ntiles*128][H]
  float* yf;                  // PHASE 4: weighted rows [ntiles*32][H] in fp32 (one rounding only, in the combine)
  int* status;
  const float* rowscale;      // PHASE 3: 1 / g_t of every term row of the x operand [ntiles*128] (0 on padding rows)
  float act_g1;               // PHASE 3/4: global scale of the first term of the SiLU*mul activations
  int NBLK, KB, KT, KB2, H;
  int dbg;                    // ablation build only (-DB200_PF_ABLATE): 1 epilogue without math, 2 no MMAs, 4 no scale moves, 8 one weight producer, bits 8-11 ring depth cap
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
    const float gs_in = P.gs_in;
    for (long long w = blockIdx.x; w < nwork; w += gridDim.x) {
      const int t = (int)(w / NBLK), nblk = (int)(w % NBLK);
      const int e = P.tile_expert[t];
      if (!mbar_wait(&S.acc_full[ab], aph[ab], &S.abort_flag)) *P.status = 7;
      tc_fence_after();
      const uint32_t taddr = tm_acc + 128 * ab + ((uint32_t)(warp * 32) << 16);
      if (PHASE == 1) {
        // columns 0..63 = up, 64..127 = gate of intermediate columns 64*nblk..; SiLU*mul, re-quantise 4 blocks of 16
        const float s = P.alpha[e] / gs_in;
        const float gs_out = P.gs_out;
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

// ------------------------------------------------------------------------------------------------ grouped GEMM, A resident
// The same GEMM with the activation tile kept in shared memory: a CTA takes a contiguous range of (row tile, column
// block) items, so the KB records of a row tile are fetched once and only the weight records stream (one 18 KB record
// per K box through a ring of NSB stages). That halves the L2 traffic per flop of the kernel above, which re-reads the
// activation record with every weight record. The next row tile's records replace the current ones box by box as the
// last column block of the tile releases them, so there is no drain between row tiles.
// Warps 0-7: epilogue (two per TMEM lane quadrant, each half of the columns); 8-11: scale warps (scale tiles shared
// memory -> registers -> TMEM, one warp per lane quadrant); 12: MMA issuer (converged warp, one elected lane);
// 13: producer of activation records; 14, 15: producers of weight records (alternate records: one thread issues at most
// ~3 M bulk copies per second, less than the record rate the MMAs can take).
constexpr int kPrThreads = 16 * 32;

struct PrShared {
  uint64_t a_full[12], a_empty[12], a_sfr[12];   // per K box of the resident activation tile
  uint64_t b_full[12], b_empty[12], b_sfr[12];   // per ring stage of weight records
  uint64_t acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
};

static_assert(sizeof(PrShared) <= 1024, "the epilogue's store patches start 1024 bytes after the barriers");

// PAIR: two CTAs of a cluster (an SM pair) take two row tiles of one expert and run them as ONE 256-row MMA per weight
// record (tcgen05 cta_group::2): CTA r keeps its own tile's records resident and streams only its half of every weight
// record - code rows 64r..64r+63 plus the record's scale tiles (both CTAs need the B scales of all 128 rows in their own
// TMEM), 10 KB instead of 18 KB - so a weight byte fetched from L2 feeds twice the math.
// Every load is an ordinary per-CTA bulk copy (nothing is multicast). The even CTA issues the MMAs and
// its commits arrive on both CTAs' barriers; the scale warps and epilogue warps of the odd CTA arrive on the even CTA's
// barriers across the cluster. The tile plan gives every expert an even number of tiles in this mode.
template <int PHASE, bool PAIR>
__global__ void __launch_bounds__(kPrThreads, 1) k_prefill_gemm_r(const __grid_constant__ PrefillParams P, int NSB) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int KB = P.KB, NBLK = P.NBLK;
  constexpr int kARec = PHASE >= 3 ? kMidRec : kRec;            // bytes of one operand record
  constexpr int kACodes = PHASE >= 3 ? 8192 : 16384;            // ... of which codes; the scale tiles follow
  constexpr int kARows = PHASE >= 3 ? 64 : 128;                 // operand rows per tile
  constexpr int kBSlot = kRec;                                  // bytes of a ring stage
  static_assert(!PAIR || PHASE <= 2, "the CTA-pair form exists for the W4A4 phases");
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;          // CTA of the pair; 0 issues the MMAs
  uint8_t* abuf = smem;                      // KB records of the current row tile
  uint8_t* ring = smem + ((KB * kARec + 1023) & ~1023);   // NSB weight stages
  PrShared& S = *reinterpret_cast<PrShared*>(ring + ((NSB * kBSlot + 1023) & ~1023));
  uint8_t* stage = reinterpret_cast<uint8_t*>(&S) + 1024;   // PHASE 2: eight 32-row x 144-byte patches for the epilogue's transposed stores
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid == 0) {
    const int nsf = PAIR ? 8 : 4, nep = PAIR ? 16 : 8;   // arrivals of the scale warps / epilogue warps of one or both CTAs
    for (int k = 0; k < KB; ++k) { mbar_init(&S.a_full[k], 1); mbar_init(&S.a_empty[k], 1); mbar_init(&S.a_sfr[k], nsf); }
    for (int s = 0; s < NSB; ++s) { mbar_init(&S.b_full[s], 1); mbar_init(&S.b_empty[s], 1); mbar_init(&S.b_sfr[s], nsf); }
    for (int b = 0; b < 2; ++b) { mbar_init(&S.acc_full[b], 1); mbar_init(&S.acc_empty[b], nep); }
    S.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 12) {
    if (PAIR) { tmem_alloc2(&S.tmem_base, 512); tmem_relinquish2(); }
    else { tmem_alloc(&S.tmem_base, 512); tmem_relinquish(); }
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the peer's barriers exist before anything arrives on them
  tc_fence_after();
  // arrive on barrier `bar` of the CTA that issues the MMAs: this CTA, or the even CTA of the pair across the cluster
  auto arrive_at_issuer = [&](uint64_t* bar) {
    if (!PAIR || rank == 0) mbar_arrive(bar);
    else mbar_arrive_cluster(mapa_shared(smem_u32(bar), 0));
  };
  const uint32_t tmem = S.tmem_base;
  const uint32_t tm_acc = tmem, tm_sfa = tmem + 256, tm_sfb = tmem + 256 + 16 * KB;   // 2 x 128 | KB x 16 | NSB x 16
  // This CTA's work: segments (row tile t, column blocks [n0, n1)). Whole tiles are dealt round-robin for as many full
  // rounds as there are (tiles t and t + 1 of one expert then run on neighbouring CTAs at the same time and in the same
  // block order, so the second reader of a weight record finds it in L2); the tiles left over are cut into equal ranges
  // of column blocks so that every CTA gets a share of them.
  // (PAIR: the unit is a pair of tiles (2u, 2u + 1) and the worker a cluster; this CTA's tile of unit u is 2u + rank.)
  constexpr int kPer = PAIR ? 2 : 1;
  const int NT = P.ntiles[0] / kPer, G = (int)gridDim.x / kPer, cta = (int)blockIdx.x / kPer;
  const int rounds = NT / G, T0 = rounds * G;
  const int rem = (NT - T0) * NBLK, per = (rem + G - 1) / G;
  const int ra = min(rem, cta * per), rb = min(rem, ra + per);
  auto for_each_segment = [&](auto&& body) {   // body(t, n0, n1, ordinal)
    int ord = 0;
    for (int r = 0; r < rounds; ++r) body((r * G + cta) * kPer + (int)rank, 0, NBLK, ord++);
    for (int a2 = ra; a2 < rb;) {
      const int t = (T0 + a2 / NBLK) * kPer + (int)rank, n0 = a2 % NBLK, n1 = min(NBLK, n0 + (rb - a2));
      body(t, n0, n1, ord++);
      a2 += n1 - n0;
    }
  };
  const int nkt_last = P.KT - 4 * (KB - 1);

  if (warp == 13) {
    // ============================================================== activation records: once per segment, box by box
    if (lane == 0) {
      for_each_segment([&](int t, int, int, int ord) {
        for (int kb = 0; kb < KB; ++kb) {
          if (ord >= 1 && !mbar_wait(&S.a_empty[kb], (uint32_t)((ord - 1) & 1), &S.abort_flag)) *P.status = 2;
          mbar_expect_tx(&S.a_full[kb], kARec);
          bulk_load(abuf + kb * kARec, P.arec + ((long long)t * KB + kb) * kARec, kARec, &S.a_full[kb]);
        }
      });
    }
    __syncwarp();
  } else if (warp == 14 || warp == 15) {
    // ============================================================== weight records: one per (item, K box); the two producers
    // walk the same sequence and issue alternate positions
    if (lane == 0) {
      int slot = 0, use = 0;
      bool mine = warp == 14;
      const bool solo = PF_ABLATE(8);   // diagnostic build: warp 14 issues every record, warp 15 none
      for_each_segment([&](int t, int n0, int n1, int) {
        const uint8_t* src = P.wrec + ((long long)P.tile_expert[t] * NBLK + n0) * KB * kRec;
        for (int i = 0; i < (n1 - n0) * KB; ++i) {   // the records of consecutive column blocks of an expert are contiguous
          if (mine) {
            if (use >= 1 && !mbar_wait(&S.b_empty[slot], (uint32_t)((use - 1) & 1), &S.abort_flag)) *P.status = 2;
            // PAIR: this CTA's 64 code rows of the record (rows are 128 bytes, 8-row groups contiguous) and all of its scale
            // tiles, in ONE copy (a CTA cannot issue copies faster than records arrive otherwise): the odd CTA's rows and the
            // scale tiles are the record's last 10 KB; the even CTA's rows are its first 8 KB, so it takes the whole record
            // and leaves the middle unused.
            const int skip = PAIR && rank == 1 ? 8192 : 0;
            mbar_expect_tx(&S.b_full[slot], kRec - skip);
            bulk_load(ring + slot * kBSlot, src + (long long)i * kRec + skip, kRec - skip, &S.b_full[slot]);
          }
          if (!solo) mine = !mine;
          if (++slot == NSB) { slot = 0; ++use; }
        }
      });
    }
    __syncwarp();
  } else if (warp >= 8 && warp < 12) {
    // ============================================================== scale warps
    const uint32_t lane_base = (uint32_t)((warp - 8) * 32) << 16;
    const uint32_t a_u = smem_u32(abuf) + kACodes + lane * 16, b_u = smem_u32(ring) + (PAIR && rank == 1 ? 8192 : 16384) + lane * 16;
    auto put = [&](uint32_t src, uint32_t dst_col) {   // four 512-byte scale tiles -> 16 TMEM columns of this quadrant
      uint32_t r[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 t4 = lds128(src + j * 512);
        r[4 * j] = t4.x, r[4 * j + 1] = t4.y, r[4 * j + 2] = t4.z, r[4 * j + 3] = t4.w;
      }
      tmem_st_32x32b_x16(dst_col + lane_base, r);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
    };
    int slot = 0;
    uint32_t ph = 0;
    for_each_segment([&](int, int n0, int n1, int ord) {
      for (int n = n0; n < n1; ++n)
        for (int kb = 0; kb < KB; ++kb) {
          if (n == n0) {
            if (!mbar_wait(&S.a_full[kb], (uint32_t)(ord & 1), &S.abort_flag)) *P.status = 1;
            put(a_u + kb * kARec, tm_sfa + 16 * kb);
            if (lane == 0) arrive_at_issuer(&S.a_sfr[kb]);
          }
          if (!mbar_wait(&S.b_full[slot], ph, &S.abort_flag)) *P.status = 1;
          if (!PF_ABLATE(4)) put(b_u + slot * kBSlot, tm_sfb + 16 * slot);
          if (lane == 0) arrive_at_issuer(&S.b_sfr[slot]);
          if (++slot == NSB) { slot = 0; ph ^= 1u; }
        }
    });
  } else if (warp == 12) {
    // ============================================================== MMA issuer (PAIR: of the even CTA only)
    const uint32_t el = elect_one();
    const uint32_t idesc = PAIR ? idesc_mxf4nvf4_pair(128) : idesc_mxf4nvf4(128, 128);
    const uint64_t desc0 = smem_desc_sw128_kmajor(0);
    const uint32_t a16 = smem_u32(abuf) >> 4, b16 = smem_u32(ring) >> 4;
    int slot = 0, ab = 0, works = 0;
    uint32_t ph = 0;
    uint32_t aph[2] = {0, 0};
    auto wait_ready = [&](uint64_t* bar, uint32_t parity) {   // arrivals may come from the peer CTA (see mbar_arrive_cluster)
      return mbar_wait(bar, parity, &S.abort_flag);
    };
    if (!PAIR || rank == 0)
    for_each_segment([&](int, int n0, int n1, int ord) {
      for (int n = n0; n < n1; ++n) {
        const bool first = n == n0, last = n == n1 - 1;
        if (works >= 2 && !wait_ready(&S.acc_empty[ab], aph[ab] ^ 1u)) *P.status = 5;
        for (int kb = 0; kb < KB; ++kb) {
          if (first && !wait_ready(&S.a_sfr[kb], (uint32_t)(ord & 1))) *P.status = 8;
          if (!wait_ready(&S.b_sfr[slot], ph)) *P.status = 8;
          tc_fence_after();
          const uint64_t ad = desc0 | (uint64_t)(a16 + kb * (kARec >> 4)), bd = desc0 | (uint64_t)(b16 + slot * (kBSlot >> 4));
          const int nkt = kb == KB - 1 ? nkt_last : 4;
#pragma unroll
          for (int jj = 0; jj < 4; ++jj)
            if (jj < nkt && !PF_ABLATE(2)) {
              if (PAIR)
                umma2_mxf4nvf4_p(tm_acc + 128 * ab, ad + 2 * jj, bd + 2 * jj, idesc, tm_sfa + 16 * kb + 4 * jj, tm_sfb + 16 * slot + 4 * jj,
                                 (kb > 0 || jj > 0) ? 1u : 0u, el);
              else
                umma_mxf4nvf4_p(tm_acc + 128 * ab, ad + 2 * jj, bd + 2 * jj, idesc, tm_sfa + 16 * kb + 4 * jj, tm_sfb + 16 * slot + 4 * jj,
                                (kb > 0 || jj > 0) ? 1u : 0u, el);
            }
          if (PAIR) {   // one commit frees the stage (and, after a tile's last block, the operand box) in both CTAs
            umma2_commit_p(&S.b_empty[slot], (uint16_t)3, el);
            if (last) umma2_commit_p(&S.a_empty[kb], (uint16_t)3, el);
          } else {
            umma_commit_p(&S.b_empty[slot], el);
            if (last) umma_commit_p(&S.a_empty[kb], el);   // the next segment's record of this box may land
          }
          if (++slot == NSB) { slot = 0; ph ^= 1u; }
        }
        if (PAIR) umma2_commit_p(&S.acc_full[ab], (uint16_t)3, el);
        else umma_commit_p(&S.acc_full[ab], el);
        aph[ab] ^= 1u;
        ab ^= 1;
        ++works;
      }
    });
  } else {
    // ============================================================== epilogue: thread = accumulator row, warp pair = column halves
    const int quad = warp & 3, half = warp >> 2;
    const int row = quad * 32 + lane;
    int ab = 0;
    uint32_t aph[2] = {0, 0};
    const float gs_in = PHASE <= 2 ? P.gs_in : 1.0f;
    const float gs_out = PHASE == 1 ? P.gs_out : 0.f;
    for_each_segment([&](int t, int n0, int n1, int) {
      // per segment: the tile's expert and (FC2) this row's pair, fetched once
      float s = P.alpha[P.tile_expert[t]] / gs_in;   // FC1: alpha / gs_in; FC2: that times the row's routing weight (0 on padding rows)
      int pr = -1;
      float rs = 0.f;   // W4A16 phases: 1 / g_t of this operand row's term
      if (PHASE == 2 || (PHASE == 4 && row < kARows)) {
        pr = P.row_pair[(long long)t * kARows + row];
        s = pr >= 0 ? s * P.wts[pr] : 0.f;
      }
      if (PHASE == 3 && row < kARows) rs = P.rowscale[(long long)t * kARows + row];
      if (PHASE == 4) {
        float g = P.act_g1;
        for (int q = 0; q < (lane & 3); ++q) g *= 6.0f;
        rs = 1.0f / g;
      }
      for (int n = n0; n < n1; ++n) {
        if (!mbar_wait(&S.acc_full[ab], aph[ab], &S.abort_flag)) *P.status = 7;
        tc_fence_after();
        const uint32_t taddr = tm_acc + 128 * ab + ((uint32_t)(quad * 32) << 16);
        if (PF_ABLATE(1)) {
        } else if (PHASE == 1) {
          // columns 0..63 = up, 64..127 = gate of intermediate columns 64*n..; SiLU*mul, re-quantise blocks of 16
          uint8_t* dst = P.orec + ((long long)t * P.KB2 + (n >> 2)) * kRec;
          uint32_t sfw = 0;
#pragma unroll
          for (int bb = 0; bb < 2; ++bb) {
            const int blk = 2 * half + bb;
            uint32_t up[16], gt[16];
            tmem_ld_32x32b_x16(taddr + 16 * blk, up);
            tmem_ld_32x32b_x16(taddr + 64 + 16 * blk, gt);
            tmem_ld_wait();
            float a[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float g = __uint_as_float(gt[i]) * s, u = __uint_as_float(up[i]) * s;
              a[i] = __fdividef(g, 1.0f + __expf(-g)) * u;
            }
            uint2 pk;
            const uint8_t sb = quantize_block16(a, gs_out, pk);
            *reinterpret_cast<uint2*>(dst + rec_code_offset(row, 4 * (n & 3) + blk)) = pk;
            sfw |= (uint32_t)sb << (8 * bb);
          }
          *reinterpret_cast<uint16_t*>(dst + 16384 + (n & 3) * 512 + (row & 31) * 16 + (row >> 5) * 4 + 2 * half) = (uint16_t)sfw;
        } else if (PHASE >= 3 && quad >= 2) {
          // accumulator rows 64..127 of the W4A16 phases belong to no operand row
        } else if (PHASE == 3) {
          // W4A16 FC1: rows 4p..4p+3 are the four terms of pair p, each scaled by its 1/g_t. This warp holds two 16-column
          // blocks of the pair; lanes 0,1 of the pair's four end up with the sums of the first block and lanes 2,3 with
          // those of the second (an exchange across the lane pairs, then one add inside them), so that SiLU*mul and the
          // expansion of the activations into four terms run once per block: the even lane of each lane pair does it
          // and writes all four term rows 4p..4p+3 of FC2's operand record.
          uint8_t* dst = P.orec + ((long long)t * P.KB2 + (n >> 2)) * kMidRec;
          uint32_t upr[2][16], gtr[2][16];
#pragma unroll
          for (int bb = 0; bb < 2; ++bb) {
            tmem_ld_32x32b_x16(taddr + 16 * (2 * half + bb), upr[bb]);
            tmem_ld_32x32b_x16(taddr + 64 + 16 * (2 * half + bb), gtr[bb]);
          }
          tmem_ld_wait();
          const int tq = lane & 3, bsel = tq >> 1;
          float a[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float u0 = __uint_as_float(upr[0][i]) * rs, u1 = __uint_as_float(upr[1][i]) * rs;
            const float g0 = __uint_as_float(gtr[0][i]) * rs, g1v = __uint_as_float(gtr[1][i]) * rs;
            float ku = bsel ? u1 : u0, kg = bsel ? g1v : g0;
            ku += __shfl_xor_sync(0xffffffffu, bsel ? u0 : u1, 2);   // the lane two over keeps the other block and sends this one
            kg += __shfl_xor_sync(0xffffffffu, bsel ? g0 : g1v, 2);
            ku += __shfl_xor_sync(0xffffffffu, ku, 1);
            kg += __shfl_xor_sync(0xffffffffu, kg, 1);
            kg *= s, ku *= s;
            a[i] = __fdividef(kg, 1.0f + __expf(-kg)) * ku;
          }
          if ((tq & 1) == 0) {
            uint2 codes[kTerms];
            uint8_t sf[kTerms];
            if (expand_block16(a, P.act_g1, codes, sf)) P.status[1] = 1;   // beyond the range of the fixed activation scale
            const int blk = 2 * half + bsel, r0 = row & ~3;
#pragma unroll
            for (int q = 0; q < kTerms; ++q) {
              *reinterpret_cast<uint2*>(dst + rec_code_offset(r0 + q, 4 * (n & 3) + blk)) = codes[q];
              dst[8192 + (n & 3) * 512 + ((r0 + q) & 31) * 16 + ((r0 + q) >> 5) * 4 + blk] = sf[q];
            }
          }
        } else if (PHASE == 4) {
          // W4A16 FC2: the four term rows of a pair are scaled and added; lane t of the pair stores columns 16t..16t+15 of
          // this warp's 64-column half, so the four lanes write one contiguous 128-byte segment of the pair's row.
          uint32_t r[4][16];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x16(taddr + 64 * half + 16 * c, r[c]);
          tmem_ld_wait();
          // reduce-scatter over the pair's four lanes: lane tq ends up with the sums of chunk tq only
          const int tq = lane & 3, hi = tq >> 1, lo = tq & 1;
          float o[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float k2[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const float mine = __uint_as_float(hi ? r[2 + j][i] : r[j][i]) * rs, other = __uint_as_float(hi ? r[j][i] : r[2 + j][i]) * rs;
              k2[j] = mine + __shfl_xor_sync(0xffffffffu, other, 2);   // the lane two over keeps the other two chunks and sends these
            }
            const float keep = lo ? k2[1] : k2[0], send = lo ? k2[0] : k2[1];
            o[i] = (keep + __shfl_xor_sync(0xffffffffu, send, 1)) * s;
          }
          if (pr >= 0) {
            float* yrow = P.yf + ((long long)t * 16 + (row >> 2)) * P.H + 128 * n + 64 * half + 16 * tq;
#pragma unroll
            for (int i = 0; i < 4; ++i) *reinterpret_cast<float4*>(yrow + 4 * i) = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
          }
        } else {
          // This thread holds 64 bf16 of its row (128 bytes); the warp transposes its 32 x 128-byte block through its own
          // patch of shared memory so that every store instruction writes whole 128-byte row segments (four rows per
          // instruction) instead of 32 scattered 16-byte pieces.
          uint32_t r[4][16];
#pragma unroll
          for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x16(taddr + 64 * half + 16 * c, r[c]);
          tmem_ld_wait();
          uint8_t* patch = stage + warp * (32 * 144);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[c][2 * i]) * s, __uint_as_float(r[c][2 * i + 1]) * s);
              o[i] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(patch + lane * 144 + 32 * c) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(patch + lane * 144 + 32 * c + 16) = make_uint4(o[4], o[5], o[6], o[7]);
          }
          __syncwarp();
          const unsigned valid = __ballot_sync(0xffffffffu, pr >= 0);   // bit l: row quad*32 + l holds a pair
          __nv_bfloat16* ybase = P.y + ((long long)t * 128 + quad * 32) * P.H + 128 * n + 64 * half;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int rr = 4 * j + (lane >> 3);   // row of the warp's block this lane stores a 16-byte chunk of
            const uint4 v4 = *reinterpret_cast<const uint4*>(patch + rr * 144 + (lane & 7) * 16);
            if ((valid >> rr) & 1u) *reinterpret_cast<uint4*>(ybase + (long long)rr * P.H + (lane & 7) * 8) = v4;
          }
          __syncwarp();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_at_issuer(&S.acc_empty[ab]);
        aph[ab] ^= 1u;
        ab ^= 1;
      }
    });
  }
  tc_fence_before();
  __syncthreads();
  if (PAIR) cluster_sync_all();   // the pair's last MMAs read both CTAs' shared memory and write both CTAs' TMEM
  if (warp == 12) {
    if (PAIR) tmem_dealloc2(tmem, 512);
    else tmem_dealloc(tmem, 512);
  }
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

// the same from fp32 rows (W4A16 path: the only bf16 rounding of the layer is this one)
__global__ void __launch_bounds__(256) k_combine_f32(const float* __restrict__ y, const int* __restrict__ dst_row, int M, int top_k, int H,
                                                     __nv_bfloat16* __restrict__ out) {
  const int chunks = H / 8;
  const long long total = (long long)M * chunks;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int tok = (int)(i / chunks), c = (int)(i % chunks);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int j = 0; j < top_k; ++j) {
      const int r = dst_row[tok * top_k + j];
      if (r < 0) continue;   // empty slot
      const float4 a = *reinterpret_cast<const float4*>(y + (long long)r * H + c * 8), b = *reinterpret_cast<const float4*>(y + (long long)r * H + c * 8 + 4);
      acc[0] += a.x, acc[1] += a.y, acc[2] += a.z, acc[3] += a.w, acc[4] += b.x, acc[5] += b.y, acc[6] += b.z, acc[7] += b.w;
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
  long long experts, offsets, pairs, route_ws, ntiles, tile_expert, tile_tab, row_pair, dst_row, status, xrec, arec, y, total;
  int max_tiles;
};

static inline long long pf_align(long long v) { return (v + 255) / 256 * 256; }

static PrefillLayout prefill_layout(int E, int H, int I, int top_k, int max_tokens) {
  PrefillLayout L;
  const long long P = (long long)max_tokens * top_k;
  const int KB1 = (H + 255) / 256, KB2 = (I + 255) / 256;
  L.max_tiles = (int)(P / 128 + 2 * E);   // every expert may end in a partly filled tile, plus one empty tile to make its count even
  long long o = 0;
  L.experts = o, o = pf_align(o + 4LL * E);
  L.offsets = o, o = pf_align(o + 4LL * (E + 1));
  L.pairs = o, o = pf_align(o + 4 * P);
  L.route_ws = o, o = pf_align(o + b200moe_route_workspace_bytes((int)P, E));
  L.ntiles = o, o += 256;
  L.tile_expert = o, o = pf_align(o + 4LL * L.max_tiles);
  L.tile_tab = o, o = pf_align(o + 8LL * L.max_tiles);   // tile_first [max_tiles], then tile_end [max_tiles]
  L.row_pair = o, o = pf_align(o + 4LL * L.max_tiles * 128);
  L.dst_row = o, o = pf_align(o + 4 * P);
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

// Byte offsets of the tables and records inside a prefill workspace, for tools and tests that read them back:
// out[0..11] = experts, offsets, pairs, ntiles, tile_expert, tile_first, tile_end, row_pair, dst_row, x records, activation
// records, weighted rows; out[12] = tile capacity, out[13] = total bytes.
void b200_prefill_workspace_map(int E, int H, int I, int top_k, int max_tokens, long long* out) {
  const PrefillLayout L = prefill_layout(E, H, I, top_k, max_tokens);
  const long long v[14] = {L.experts, L.offsets, L.pairs, L.ntiles, L.tile_expert, L.tile_tab, L.tile_tab + 4LL * L.max_tiles, L.row_pair,
                           L.dst_row, L.xrec, L.arec, L.y, L.max_tiles, L.total};
  for (int i = 0; i < 14; ++i) out[i] = v[i];
}

// One GEMM launch. Phases 1/2 (W4A4): the resident-A kernel when the row tile's KB records plus at least 3 weight stages fit
// in shared memory and the scale columns fit in TMEM, otherwise the kernel that streams both operands. Phases 3/4 (W4A16)
// exist for the resident-A kernel only.
// B200MOE_PREFILL_PAIR=1: the W4A4 GEMMs run as CTA pairs (256 rows per weight record, cta_group::2). Correct (the parity
// tests run in both modes) but off by default: per row tile it is as fast as the single-CTA form, not faster, and the tile
// plan must give every expert an even number of tiles (+20 % tiles at 4096 tokens over 128 experts, +11 % at 8192).
// Measured at 4096 tokens: FC1 116 us as pairs against 98 us, FC2 73 us against 60 us. Why pairing does not pay as built:
// both CTAs' ring stages must sit at the same shared-memory offsets (one B descriptor serves both), the even CTA's code rows
// and the scale tiles are the two ends of a record, so a stage is 18 KB in both CTAs and FC1 (144 KB of resident
// activations) keeps four stages - and a stage's round trip (copy, scale move, MMA, commit back across the cluster) is longer
// for a pair; FC2 is bound by its epilogue and its bf16 rows, which pairing does not change. Two copies of 8 + 2 KB per CTA
// and record allow seven 10 KB stages but run into the rate at which an SM accepts bulk copies (same total time).
// Barrier arrivals across the cluster use default (CTA-scope) semantics; with release/acquire at cluster scope every
// arrival and every poll took about a microsecond and the pair form was 2.3 times slower than the single-CTA form.
static bool pair_mode_enabled() {
  static const bool on = [] { const char* c = getenv("B200MOE_PREFILL_PAIR"); return c && c[0] == '1'; }();
  return on;
}

// Whether the W4A4 GEMMs of this shape run as CTA pairs: both phases' resident tiles and at least 3 ring stages must fit.
static bool prefill_pairs(int H, int I) {
  const int KB1 = (H + 255) / 256, KB2 = (I + 255) / 256;
  if (!pair_mode_enabled() || KB1 > 12 || KB2 > 12) return false;
  const int a1 = KB1 * kRec, n1 = (227 * 1024 - 3072 - 256 - a1) / kRec;   // as launch_gemm sizes the FC1 ring
  return n1 >= 3 && (512 - 256 - 16 * KB1) / 16 >= 3;
}

static int launch_gemm(const PrefillParams& p, int phase, int KB, int sms, bool pair, cudaStream_t st) {
  const int tail = 1024 + ((phase == 2) ? 8 * 32 * 144 : 0);   // barriers (+ the W4A4 FC2 epilogue's store patches)
  const int abytes = (KB * (phase >= 3 ? kMidRec : kRec) + 1023) & ~1023;   // the resident operand tile
  const int slot_bytes = kRec;
  int nsb = (227 * 1024 - 2048 - tail - 256 - abytes) / slot_bytes;
  const int tmem_cap = (512 - 256 - 16 * KB) / 16;
  if (nsb > tmem_cap) nsb = tmem_cap;
  if (nsb > 12) nsb = 12;
  // W4A4 FC2 (three K boxes per tile): five stages measure faster than the seven that fit (57.7 us against 62.5 at 4096
  // tokens, 102 against 109 at 8192; six: 63.1, four: 59.1); DRAM traffic is at its minimum either way, so the cause is not
  // re-reads and is not known. The W4A16 FC2 likewise (27.6 us against 29.3 at 128 tokens over 128 experts).
  if ((phase == 2 || phase == 4) && !pair && nsb > 5) nsb = 5;
#ifdef B200_PF_ABLATE
  if (((p.dbg >> 8) & 15) >= 2 && ((p.dbg >> 8) & 15) < nsb) nsb = (p.dbg >> 8) & 15;   // ring depth cap
#endif
  if (KB <= 12 && nsb >= 3) {
    const int sm_r = 1024 + abytes + ((nsb * slot_bytes + 1023) & ~1023) + tail;
    const void* fn = pair ? (phase == 1 ? (const void*)k_prefill_gemm_r<1, true> : (const void*)k_prefill_gemm_r<2, true>)
                   : phase == 1 ? (const void*)k_prefill_gemm_r<1, false> : phase == 2 ? (const void*)k_prefill_gemm_r<2, false>
                   : phase == 3 ? (const void*)k_prefill_gemm_r<3, false> : (const void*)k_prefill_gemm_r<4, false>;
    if (pair && phase > 2) return B200MOE_ERR_SHAPE;
    static thread_local int configured_r[6] = {0, 0, 0, 0, 0, 0};
    const int ci = pair ? 3 + phase : phase - 1;
    if (configured_r[ci] < sm_r) {
      B200_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, sm_r));
      configured_r[ci] = sm_r;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(pair ? (sms & ~1) : sms), cfg.blockDim = dim3(kPrThreads), cfg.dynamicSmemBytes = (size_t)sm_r, cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr, cfg.numAttrs = pair ? 1 : 0;
    PrefillParams pp = p;
    void* args[] = {(void*)&pp, (void*)&nsb};
    B200_CUDA_TRY(cudaLaunchKernelExC(&cfg, fn, args));
  } else {
    if (phase > 2 || pair) return B200MOE_ERR_SHAPE;
    const int smem = 1024 + kPfStages * 2 * kRec + (int)sizeof(PfShared);
    static thread_local bool configured = false;
    if (!configured) {
      B200_CUDA_TRY(cudaFuncSetAttribute(k_prefill_gemm<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      B200_CUDA_TRY(cudaFuncSetAttribute(k_prefill_gemm<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      configured = true;
    }
    if (phase == 1) k_prefill_gemm<1><<<sms, kPfThreads, smem, st>>>(p);
    else k_prefill_gemm<2><<<sms, kPfThreads, smem, st>>>(p);
  }
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// w1t / w2t: the weight tile records of b200moe_layer_prepack. gs_x / gs_a: global scales of the two activation quantisations.
// Launches: router (3) -> row map (tile plan fused) -> token-major quantiser -> FC1 GEMM -> FC2 GEMM -> combine.
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
  int* tile_first = (int*)(w + L.tile_tab);
  int* tile_end = tile_first + L.max_tiles;
  int* row_pair = (int*)(w + L.row_pair);
  int* dst_row = (int*)(w + L.dst_row);
  int* status = (int*)(w + L.status);
  if (Umax > 256) return B200MOE_ERR_LIMIT;
  int rc = b200moe_route(ids, P, E, Umax, experts, offsets, pairs, w + L.route_ws, L.total - L.route_ws, st);
  if (rc != B200MOE_OK) return rc;
  const bool pair = prefill_pairs(H, I) && sms >= 2;
  const int max_tiles = P / 128 + 2 * Umax;   // tiles this batch can need (<= the workspace's capacity)
  {
    const int rows = max_tiles * 128;
    int grid = (rows + 255) / 256;
    if (grid > sms * 8) grid = sms * 8;
    k_prefill_rowmap<<<grid, 256, 0, st>>>(ids, P, experts, offsets, pairs, Umax, max_tiles, KB1, pair ? 1 : 0, ntiles, tile_expert, tile_first, tile_end,
                                           w + L.xrec, row_pair, dst_row);
    B200_LAUNCH_CHECK();
  }
  k_quantize_scatter<<<M, 128, 0, st>>>((const __nv_bfloat16*)x, dst_row, M, H, KB1, top_k, gs_x, w + L.xrec);
  B200_LAUNCH_CHECK();
  PrefillParams p;
  memset(&p, 0, sizeof(p));
  p.ntiles = ntiles, p.tile_expert = tile_expert, p.row_pair = row_pair, p.status = status, p.H = H;
#ifdef B200_PF_ABLATE
  p.dbg = getenv("B200MOE_PF_ABLATE") ? atoi(getenv("B200MOE_PF_ABLATE")) : 0;
#endif
  // FC1
  p.arec = w + L.xrec, p.wrec = w1t, p.alpha = alpha1, p.gs_in = gs_x, p.gs_out = gs_a, p.orec = w + L.arec;
  p.NBLK = I / 64, p.KB = KB1, p.KT = KT1, p.KB2 = KB2;
  rc = launch_gemm(p, 1, KB1, sms, pair, st);
  if (rc != B200MOE_OK) return rc;
  // FC2
  p.arec = w + L.arec, p.wrec = w2t, p.alpha = alpha2, p.gs_in = gs_a, p.gs_out = 0.f, p.orec = nullptr;
  p.wts = wts, p.y = (__nv_bfloat16*)(w + L.y);
  p.NBLK = H / 128, p.KB = KB2, p.KT = KT2;
  rc = launch_gemm(p, 2, KB2, sms, pair, st);
  if (rc != B200MOE_OK) return rc;
  k_prefill_combine<<<sms * 8, 256, 0, st>>>((const __nv_bfloat16*)(w + L.y), dst_row, M, top_k, H, (__nv_bfloat16*)out);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

int b200_prefill_status_offset(int E, int H, int I, int top_k, int max_tokens, long long* off) {
  *off = prefill_layout(E, H, I, top_k, max_tokens).status;
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// W4A16 layer call for mid-sized batches (the decode path's arithmetic, one pass over the touched experts' weights).
struct MidLayout {
  long long experts, offsets, pairs, route_ws, ntiles, tile_expert, tile_tab, row_pair, rowscale, dst_row, tok_amax, status, xrec, arec, y, total;
  int max_tiles;
};

static MidLayout mid_layout(int E, int H, int I, int top_k, int max_tokens) {
  MidLayout L;
  const long long P = (long long)max_tokens * top_k;
  const int KB1 = (H + 255) / 256, KB2 = (I + 255) / 256;
  L.max_tiles = (int)(P / 16 + E);
  long long o = 0;
  L.experts = o, o = pf_align(o + 4LL * E);
  L.offsets = o, o = pf_align(o + 4LL * (E + 1));
  L.pairs = o, o = pf_align(o + 4 * P);
  L.route_ws = o, o = pf_align(o + b200moe_route_workspace_bytes((int)P, E));
  L.ntiles = o, o += 256;
  L.tile_expert = o, o = pf_align(o + 4LL * L.max_tiles);
  L.tile_tab = o, o = pf_align(o + 8LL * L.max_tiles);
  L.row_pair = o, o = pf_align(o + 4LL * L.max_tiles * 64);
  L.rowscale = o, o = pf_align(o + 4LL * L.max_tiles * 64);
  L.dst_row = o, o = pf_align(o + 4 * P);
  L.tok_amax = o, o = pf_align(o + 4LL * max_tokens);
  L.status = o, o += 256;
  L.xrec = o, o = pf_align(o + (long long)L.max_tiles * KB1 * kMidRec);
  L.arec = o, o = pf_align(o + (long long)L.max_tiles * KB2 * kMidRec);
  L.y = o, o = pf_align(o + (long long)L.max_tiles * 16 * H * 4);
  L.total = o;
  return L;
}

long long b200_mid_workspace_bytes(int E, int H, int I, int top_k, int max_tokens) { return mid_layout(E, H, I, top_k, max_tokens).total; }

int b200_mid_status_offset(int E, int H, int I, int top_k, int max_tokens, long long* off) {
  *off = mid_layout(E, H, I, top_k, max_tokens).status;
  return 0;
}

int b200_mid_forward(int E, int H, int I, int top_k, const uint8_t* w1t, const uint8_t* w2t, const float* alpha1, const float* alpha2,
                     const void* x, const int* ids, const float* wts, int M, void* out, void* ws, long long ws_bytes, int ws_tokens,
                     float act_g1, int sms, cudaStream_t st) {
  const MidLayout L = mid_layout(E, H, I, top_k, ws_tokens);
  if (ws_bytes < L.total || M > ws_tokens) return B200MOE_ERR_WORKSPACE;
  uint8_t* w = (uint8_t*)ws;
  const int P = M * top_k;
  const int Umax = E < P ? E : P;
  const int KB1 = (H + 255) / 256, KB2 = (I + 255) / 256, KT1 = (H / 16 + 3) / 4, KT2 = (I / 16 + 3) / 4;
  if (Umax > 256 || KB1 > 12) return B200MOE_ERR_LIMIT;
  int* experts = (int*)(w + L.experts);
  int* offsets = (int*)(w + L.offsets);
  int* pairs = (int*)(w + L.pairs);
  int* ntiles = (int*)(w + L.ntiles);
  int* tile_expert = (int*)(w + L.tile_expert);
  int* tile_first = (int*)(w + L.tile_tab);
  int* row_pair = (int*)(w + L.row_pair);
  float* rowscale = (float*)(w + L.rowscale);
  int* dst_row = (int*)(w + L.dst_row);
  int rc = b200moe_route(ids, P, E, Umax, experts, offsets, pairs, w + L.route_ws, L.total - L.route_ws, st);
  if (rc != B200MOE_OK) return rc;
  const int max_tiles = P / 16 + Umax;
  int* tile_end = tile_first + max_tiles;
  {
    int grid = (max_tiles * 16 * KB1 + 255) / 256;
    if (grid > sms * 4) grid = sms * 4;
    k_mid_rowmap<<<grid, 256, 0, st>>>(ids, P, experts, offsets, pairs, Umax, max_tiles, KB1, ntiles, tile_expert, tile_first, tile_end, w + L.xrec,
                                       row_pair, dst_row);
    B200_LAUNCH_CHECK();
  }
  k_expand_scatter<<<M, 128, 0, st>>>((const __nv_bfloat16*)x, dst_row, M, H, KB1, top_k, w + L.xrec, rowscale);
  B200_LAUNCH_CHECK();
  PrefillParams p;
  memset(&p, 0, sizeof(p));
  p.ntiles = ntiles, p.tile_expert = tile_expert, p.row_pair = row_pair, p.status = (int*)(w + L.status), p.H = H;
  p.rowscale = rowscale, p.act_g1 = act_g1;
#ifdef B200_PF_ABLATE
  p.dbg = getenv("B200MOE_PF_ABLATE") ? atoi(getenv("B200MOE_PF_ABLATE")) : 0;
#endif
  // FC1
  p.arec = w + L.xrec, p.wrec = w1t, p.alpha = alpha1, p.orec = w + L.arec;
  p.NBLK = I / 64, p.KB = KB1, p.KT = KT1, p.KB2 = KB2;
  rc = launch_gemm(p, 3, KB1, sms, false, st);
  if (rc != B200MOE_OK) return rc;
  // FC2
  p.arec = w + L.arec, p.wrec = w2t, p.alpha = alpha2, p.orec = nullptr;
  p.wts = wts, p.yf = (float*)(w + L.y);
  p.NBLK = H / 128, p.KB = KB2, p.KT = KT2;
  rc = launch_gemm(p, 4, KB2, sms, false, st);
  if (rc != B200MOE_OK) return rc;
  k_combine_f32<<<sms * 4, 256, 0, st>>>((const float*)(w + L.y), dst_row, M, top_k, H, (__nv_bfloat16*)out);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}
