// The decode-regime MoE layer on the 5th-generation tensor cores: weights are consumed as FP4 straight from shared
// memory by tcgen05.mma kind::mxf4nvf4 with their E4M3 block scales in TMEM - no CUDA-core dequantisation at all - so the
// SMs only move bytes and the kernel is bound by HBM. It keeps the contract of the reference's decode kernels
// (sm120fp4/kernels/{fc1_w4a16,fc1_mma,fc2_w4a16,fc2_mma_pf}.py: W4A16, fp32 accumulation, alpha in fp32, SiLU*mul,
// weighted combine, bit-identical from call to call).
//
// W4A16 on an FP4 x FP4 instruction: a 16-bit activation vector is written as a short sum of NVFP4 vectors,
//     x = q1*s1/g1 + q2*s2/g2 + q3*s3/g3 + q4*s4/g4 + r,   g_t = g1 * 6^(t-1),   |r| <= blockmax(x) * 6^-4 (about 2^-10.3),
// each term the NVFP4 quantisation (E2M1 codes, E4M3 scale per 16 values) of the residual left by the terms before it.
// The terms of a token are adjacent columns of the B operand; the epilogue adds the four accumulator columns with their
// 1/g_t. Four terms carry more mantissa than bf16 for the values that decide a dot product and keep the layer's error
// against the fp32 oracle below the bf16 output rounding.
//
// Structure: one CTA per SM = one stream-K worker. Warps 0-3: epilogue (tcgen05.ld of a double-buffered TMEM accumulator,
// term sums, SiLU*mul, re-expansion of the activations for FC2, fixed-order reduction of split units). Warps 4-7: scale
// warps, one per TMEM lane quadrant (scale tiles of a landed stage shared memory -> registers -> TMEM). Warp 8: MMA issuer
// (converged warp, one elected lane: four K=64 MMAs per 256-code tile, tcgen05.commit frees the ring stage). Warps 9-10:
// TMA producers (one bulk copy per 18 KB tile record into a shared-memory ring, FC2 tiles prefetched across the
// FC1->FC2 grid barrier). The per-tile loops of the single-thread roles are kept free of divisions: at 148 tiles per
// microsecond per GPU a role has only a few hundred cycles per tile.
#include "common.cuh"
#include "tcgen05.cuh"
#include "decode_params.h"
#include "expand.cuh"
#include <string.h>
#include <stdlib.h>

namespace b200 {

constexpr int kTcProducers = 2;    // TMA producer warps: one thread issues only ~2.5 M bulk operations per second
constexpr int kTcThreads = (4 + 4 + 1 + kTcProducers) * 32;   // epilogue warps 0-3, scale warps 4-7, MMA warp 8, producers 9..
constexpr int kTcStage = 18432;   // 16 KB codes + 2 KB scale tiles
constexpr int kTcMaxE = 256, kTcMaxP = 256;

struct TcTables {
  int ids[kTcMaxP];
  float wts[kTcMaxP];
  int cnt[kTcMaxE], base[kTcMaxE], uidx[kTcMaxE], experts[kTcMaxE];
  float colscale[64];          // 1 / g_t of every B column of the FC1 operand (token-major, four terms per token)
  float a1[kTcMaxE], a2n[kTcMaxE];   // per touched expert (unit index): alpha1, alpha2 relative to the layer's largest alpha2
  int U;
  unsigned long long gate0[2];   // arrival counts of the two FC1 gates before this launch (a multiple of the worker count)
  volatile int abort_flag;
  int last_flag;
  uint32_t tmem_base;
  uint64_t full[12], empty[12], sfr[12];   // stage landed / stage consumed / scale tiles of the stage are in TMEM
  uint64_t acc_full[2], acc_empty[2];
  uint64_t xb_full, fc1_done;   // x operand landed / this worker's FC1 MMAs are complete
};

#ifdef B200_TIMERS
#define TC_T0(var) long long var = clock64()
#define TC_ADD(acc, var) acc += clock64() - var
#define TC_TRACE(j, k) do { if (P.debug && v == 5 && (threadIdx.x & 31) == 0 && (j) < 128) P.debug[148 * 16 + (j) * 8 + (k)] = clock64() - tm_begin; } while (0)
#else
#define TC_TRACE(j, k)
#define TC_T0(var)
#define TC_ADD(acc, var)
#endif

__device__ __forceinline__ float tc_silu_mul(float gate, float up) { return __fdividef(gate, 1.0f + __expf(-gate)) * up; }

// ------------------------------------------------------------------------------------------------ x -> B operand
// One block of 128 threads per token slot (N/4 slots): token amax, then every 16-value block expanded into four NVFP4
// terms. The block is small enough (registers, shared memory) to be resident next to a block of the layer kernel.
// xb: the FC1 B operand exactly as the kernel wants it in shared memory, so that ONE bulk copy brings it in:
//   [KB1 boxes][N rows (token*4 + term)][128 B] in the 128-byte-swizzle image (16-byte chunk c of row n sits at chunk
//   c ^ (n & 7)), followed by KT1 scale tiles of 512 B (128x4 order, rows >= N zero). colscale f32 [N] = 1/g_t.
__global__ void __launch_bounds__(128, 10) k_expand_x(const __nv_bfloat16* __restrict__ x, int M, int H, int N, int KB1, uint8_t* __restrict__ xb,
                                                  float* __restrict__ colscale) {
  const int tok = blockIdx.x, tid = threadIdx.x;
  grid_launch_dependents();   // the layer kernel may start its prologue and weight prefetch now; it waits before reading xb
  grid_dependency_wait();     // this kernel is itself launched programmatically: x (and the workspace it writes) belong to
                              // whatever ran before it in the stream until that has completed
  uint8_t* xsf = xb + (long long)KB1 * N * 128;
  __shared__ float wm[4];
  __shared__ float s_g1;
  // each thread keeps its (at most two) 16-value blocks in registers: one pass over x serves the token amax and the expansion
  const int nblk = KB1 * 16;                 // blocks over the padded K (KB1 * 256 values); nblk <= 256
  uint4 raw[2][2];
  float m = 0.f;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int b = tid + 128 * j;
    raw[j][0] = raw[j][1] = make_uint4(0u, 0u, 0u, 0u);
    if (tok < M && b < nblk && b * 16 < H) {
      raw[j][0] = *reinterpret_cast<const uint4*>(x + (long long)tok * H + b * 16);
      raw[j][1] = *reinterpret_cast<const uint4*>(x + (long long)tok * H + b * 16 + 8);
      const uint32_t w[8] = {raw[j][0].x, raw[j][0].y, raw[j][0].z, raw[j][0].w, raw[j][1].x, raw[j][1].y, raw[j][1].z, raw[j][1].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) m = fmaxf(m, fmaxf(fabsf(__uint_as_float(w[i] << 16)), fabsf(__uint_as_float(w[i] & 0xffff0000u))));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((tid & 31) == 0) wm[tid >> 5] = m;
  __syncthreads();
  m = fmaxf(fmaxf(wm[0], wm[1]), fmaxf(wm[2], wm[3]));
  const float g1 = 2688.0f / fmaxf(m, 1e-30f);
  if (tid < kTerms) {
    float g = g1;
    for (int t = 0; t < tid; ++t) g *= 6.0f;
    colscale[tok * kTerms + tid] = tok < M ? 1.0f / g : 0.f;
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int b = tid + 128 * j;
    if (b >= nblk) break;
    uint2 codes[kTerms];
    uint8_t sf[kTerms];
    if (tok < M && b * 16 < H) {
      float r[16];
      const uint32_t w[8] = {raw[j][0].x, raw[j][0].y, raw[j][0].z, raw[j][0].w, raw[j][1].x, raw[j][1].y, raw[j][1].z, raw[j][1].w};
#pragma unroll
      for (int i = 0; i < 8; ++i) { r[2 * i] = __uint_as_float(w[i] << 16); r[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
      expand_block16(r, g1, codes, sf);
    } else {
#pragma unroll
      for (int t = 0; t < kTerms; ++t) { codes[t] = make_uint2(0u, 0u); sf[t] = 0; }
    }
    const int kb = b >> 4, chunk = (b & 15) >> 1, half = b & 1;   // 8 code bytes = half a 16-byte chunk
#pragma unroll
    for (int t = 0; t < kTerms; ++t) {
      const int n = tok * kTerms + t;
      *reinterpret_cast<uint2*>(xb + ((long long)kb * N + n) * 128 + ((chunk ^ (n & 7)) << 4) + half * 8) = codes[t];
      if ((b >> 2) < (H / 16 + 3) / 4) xsf[(long long)(b >> 2) * 512 + (n & 31) * 16 + (n >> 5) * 4 + (b & 3)] = sf[t];
    }
  }
}

// ------------------------------------------------------------------------------------------------ weight tiles
// Kernel-native weight layout, built once per layer: every (expert, block, K box) tile is ONE contiguous 18 KB record =
// the shared-memory image of its 128 rows x 128 B of codes (128-byte swizzle) followed by its four 512 B scale tiles, so
// a single bulk copy per tile streams it at full HBM rate (one thread issues only ~2.5 M TMA operations per second,
// whatever their size; 2-D boxes from the checkpoint layout need 3-4 operations per tile).
//   FC1 record (e, cb, kb): rows 0..63 = up rows 64cb.., rows 64..127 = gate rows I+64cb..; scale rows likewise.
//   FC2 record (e, nb, kb): rows = output rows 128nb...
__global__ void __launch_bounds__(256) k_pack_tiles(const uint8_t* __restrict__ q, const uint8_t* __restrict__ sf, uint8_t* __restrict__ out,
                                                    int E, int rows_per_expert, int row_bytes, int blocks, int KB, int KT, int fc1, int I,
                                                    long long sf_expert_stride) {
  const long long records = (long long)E * blocks * KB;
  const long long total = records * (1024 + 128);   // 1024 code chunks of 16 B + 128 scale rows x 16 B
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long rec = i / 1152;
    const int w = (int)(i % 1152);
    const int kb = (int)(rec % KB), blk = (int)((rec / KB) % blocks), e = (int)(rec / ((long long)KB * blocks));
    uint8_t* dst = out + rec * kTcStage;
    if (w < 1024) {
      const int r = w >> 3, c = w & 7;
      const int src_row = fc1 ? (r < 64 ? 64 * blk + r : I + 64 * blk + (r - 64)) : 128 * blk + r;
      const int byte = kb * 128 + c * 16;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (byte < row_bytes) v = *reinterpret_cast<const uint4*>(q + ((long long)e * rows_per_expert + src_row) * row_bytes + byte);
      *reinterpret_cast<uint4*>(dst + r * 128 + ((c ^ (r & 7)) << 4)) = v;
    } else {
      const int r = w - 1024;   // scale row of the record: four K tiles x 4 bytes
      const int src_row = fc1 ? (r < 64 ? 64 * blk + r : I + 64 * blk + (r - 64)) : 128 * blk + r;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int kt = 4 * kb + j;
        uint32_t v = 0;
        if (kt < KT)
          v = *reinterpret_cast<const uint32_t*>(sf + e * sf_expert_stride + ((long long)(src_row >> 7) * KT + kt) * 512 + (src_row & 31) * 16 +
                                                 ((src_row & 127) >> 5) * 4);
        *reinterpret_cast<uint32_t*>(dst + 16384 + j * 512 + (r & 31) * 16 + (r >> 5) * 4) = v;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------ the layer kernel
template <int NB>   // N = 16 * NB columns of the B operand (tokens x four terms): NB = 1 (M<=4), 2 (M<=8), 4 (M<=16)
__global__ void __launch_bounds__(kTcThreads, 1) k_moe_decode_tc(const __grid_constant__ DecodeTcParams P) {
  constexpr int N = 16 * NB;
  constexpr int kSlab = N * 128 + 2048;     // FC2 activation slab of one tile: N rows x 128 B codes + 4 scale tiles
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int NS = P.NS;
  uint8_t* ring = smem;                                   // NS x [16 KB codes | 2 KB scales]
  uint8_t* region = smem + NS * kTcStage;                 // FC1: resident x operand [KB1][N x 128 B] then its scale tiles;
                                                          // FC2: NS activation slabs
  TcTables& T = *reinterpret_cast<TcTables*>(region + P.region_bytes);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef B200_TIMERS
  if (tid == 0 && P.debug) { unsigned long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); P.debug[blockIdx.x * 16 + 13] = (long long)g; }
#endif
  const int npairs = P.M * P.top_k;
  const int V = gridDim.x;
  const int KB1 = P.KB1, KB2 = P.KB2, CB1 = P.CB1, NB2 = P.NB2;

  // ---------------------------------------------------------------- prologue
  // Every global load of the prologue is issued at entry, each by a thread of its own, so that their latencies overlap
  // one another and the barrier / TMEM set-up: pair p is thread p's (npairs <= 256 < threads).
  int my_e = -1;
  float my_w = 0.f;
  if (tid < npairs) { my_e = P.ids[tid]; my_w = P.wts[tid]; }
  // the per-expert scales of ALL experts come in with the ids (no load depends on another): thread e holds expert e's
  float ex_a1 = 0.f, ex_a2 = 0.f;
  if (tid < P.E) { ex_a1 = P.alpha1[tid]; ex_a2 = P.alpha2[tid]; }
  const float a2inv = P.alpha2_ref[1];
  // The gate counters are only ever incremented, by exactly V arrivals per launch and gate, and a launch starts after the
  // gates of the launch before it on this workspace have opened: whatever this thread reads, rounding down to a multiple of
  // V gives the count before this launch (other workers of this launch may have arrived already).
  unsigned long long my_gate = 0;
  if (tid == 9 * 32) my_gate = ld_acquire_gpu_u64(P.gates);
  if (tid == 10 * 32) my_gate = ld_acquire_gpu_u64(P.gates + 1);
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) { mbar_init(&T.full[s], 1); mbar_init(&T.empty[s], 1); mbar_init(&T.sfr[s], 4); }
    for (int b = 0; b < 2; ++b) { mbar_init(&T.acc_full[b], 1); mbar_init(&T.acc_empty[b], 4); }
    mbar_init(&T.xb_full, 1);
    mbar_init(&T.fc1_done, 1);
    T.abort_flag = 0;
    T.last_flag = 0;
    fence_mbar_init();
  }
  if (warp == 8) {                       // the MMA warp owns the TMEM allocation (all 512 columns: one CTA per SM)
    tmem_alloc(&T.tmem_base, 512);
    tmem_relinquish();
  }
  for (int i = tid; i < kTcMaxE; i += kTcThreads) T.cnt[i] = 0;
  if (tid < npairs) {   // a negative id marks an empty slot (expert-parallel shards mask the experts they do not own)
    if (my_e >= P.E) { *P.status = 4; my_e = -1; }
    if (my_e < 0) my_e = -1;
  }
  __syncthreads();
  if (tid < npairs) {
    T.ids[tid] = my_e;
    T.wts[tid] = my_w;
    if (my_e >= 0) atomicAdd(&T.cnt[my_e], 1);
  }
  __syncthreads();
  if (warp == 0) {
    int c[8], f[8], sc = 0, sf = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) { c[i] = T.cnt[lane * 8 + i]; f[i] = c[i] > 0; sc += c[i]; sf += f[i]; }
    int ic = sc, iff = sf;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, ic, o), b = __shfl_up_sync(0xffffffffu, iff, o);
      if (lane >= o) { ic += a; iff += b; }
    }
    int rc = ic - sc, rf = iff - sf;
#pragma unroll
    for (int i = 0; i < 8; ++i) { rc += c[i]; rf += f[i]; T.base[lane * 8 + i] = rc; T.uidx[lane * 8 + i] = rf; }
    if (lane == 31) T.U = iff;
  }
  __syncthreads();
  const int U = T.U;
  if (tid < P.E && T.cnt[tid] > 0) {   // thread e: expert e is touched -> its slot in the tables of touched experts
    const int u = T.uidx[tid] - 1;
    T.experts[u] = tid;
    T.a1[u] = ex_a1;
    T.a2n[u] = ex_a2 * a2inv;
  }
  if (tid == 9 * 32) T.gate0[0] = my_gate - my_gate % (unsigned long long)V;
  if (tid == 10 * 32) T.gate0[1] = my_gate - my_gate % (unsigned long long)V;
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // ---------------------------------------------------------------- work split (closed form, the same on every worker)
  // FC1: units q = (touched expert u, 64-column block cb), u-major; worker v takes q = v, v + V, ...: whole units (no
  // cross-CTA reduction), and all workers move through the experts in the same order, so the experts below uA (group A,
  // seven eighths of them) are finished grid-wide seven eighths of the way through FC1. Gate A opens when every worker
  // has finished its units of group A, gate B when all of FC1 is done; a worker's FC2 items of group A keep it busy
  // while gate B and the last slabs are still on their way.
  // FC2: the workers are split into NB2 groups, one per 128-row output block; inside a group, worker r takes the items
  // i = (u, kb) = r, r + W, ... in ascending order, accumulates them in one TMEM accumulator, and the group's partials are
  // added in worker order by whoever arrives last. A worker's first items belong to group A: they run while the tail of
  // FC1, gate B and the fetch of the remaining activation slabs are still in flight elsewhere.
  const int v = blockIdx.x;
  const int Q1 = U * CB1;
  const int nu1 = v < Q1 ? (Q1 - v + V - 1) / V : 0;
  const int n1 = nu1 * KB1;
  // With at most two rounds of FC1 units (Q1 <= 2V) gate A would open hardly before gate B, so it is left out (no
  // arrivals, nobody waits) and all of FC2 waits for gate B.
  const bool use_gate_a = Q1 > 2 * V;
  const int uA = use_gate_a ? (7 * U) / 8 : 0, qA = uA * CB1;
  const int nuA = v < qA ? (qA - v + V - 1) / V : 0;   // this worker's units of group A (its first ones)
  const int I2 = U * KB2;
  const int Wb = V / NB2, Wx = V % NB2;                // groups 0..Wx-1 have Wb + 1 workers
  int nb2, r2, W2, vlo2;
  if (v < Wx * (Wb + 1)) { nb2 = v / (Wb + 1); r2 = v - nb2 * (Wb + 1); W2 = Wb + 1; vlo2 = nb2 * (Wb + 1); }
  else { const int vv = v - Wx * (Wb + 1); nb2 = Wx + vv / Wb; r2 = vv % Wb; W2 = Wb; vlo2 = Wx * (Wb + 1) + (nb2 - Wx) * Wb; }
  const int n2 = r2 < I2 ? (I2 - r2 + W2 - 1) / W2 : 0;
  const int live2 = W2 < I2 ? W2 : I2;                 // workers of the group that hold a partial: ranks 0..live2-1
  const int dU2 = W2 / KB2, dK2 = W2 % KB2;            // item step W2 as (experts, K boxes)
#ifdef B200_TIMERS
  long long tm_a = 0, tm_b = 0, tm_c = 0, tm_d = 0;
  const long long tm_begin = clock64();
  if (tid == 0 && P.debug) { unsigned long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); P.debug[blockIdx.x * 16 + 15] = (long long)g;
    unsigned sm; asm volatile("mov.u32 %0, %%smid;" : "=r"(sm)); P.debug[blockIdx.x * 16 + 11] = sm; }
#endif
  const uint32_t tmem = T.tmem_base;
  const uint32_t tm_acc = tmem, tm_sfa = tmem + 128, tm_sfb = tmem + 320;   // accumulators 2 x 64 | weight scales NS x 16 (<= 192) | operand scales (<= 192)
  uint8_t* xb_sf = region + KB1 * (N * 128);   // scale tiles of the resident x operand (same bulk copy)

  if (warp >= 9) {
    // ============================================================== TMA producers (one thread each)
    // Both producers walk the worker's whole tile sequence with incremental indices (no divisions in the loop) and
    // issue the tiles whose position is theirs (position mod kTcProducers).
    if (lane == 0) {
      const int pw = warp - 9;
      const uint64_t pol = policy_evict_first();
      // (The resident B operand of FC1 is fetched by an epilogue thread: it has to wait for the expansion kernel, and a
      // producer that waited with it would leave half of the ring empty while the weights could already be streaming.)
      bool passed[2] = {!use_gate_a, false};
      int pend_slot[16], pend_idx[16], pend_g[16] = {0}, npend = 0, pend_head = 0;   // ring of 16: at most NS (<= 12) entries wait at a time
      int slot_g[12];                                                          // gate of the FC2 tile in each ring slot
      auto load_slab = [&](int slot, int idx) {   // activation slab (u, kb) of FC2: N x 128 B codes image + 4 scale tiles
        bulk_load(region + slot * kSlab, P.aslab + (long long)idx * kSlab, kSlab, &T.full[slot]);
      };
      // An activation slab may land only when (a) the gate of its expert group is open and (b) this worker's own FC1 MMAs
      // are complete: the slabs share their shared memory with the resident x operand, and their scale columns in TMEM
      // with the x operand's. Weight tiles of FC2 are prefetched regardless; only the slab loads wait.
      bool local_ok = n1 == 0;
      auto flush = [&]() {   // issue the parked slab loads whose conditions hold now
        while (pend_head < npend && local_ok && passed[pend_g[pend_head & 15]]) { load_slab(pend_slot[pend_head & 15], pend_idx[pend_head & 15]); ++pend_head; }
      };
      auto open_gate = [&](int g) {   // blocking: wait for (b) and for gate g and every gate before it; issue what waited for them
        if (!local_ok) {
          if (!mbar_wait(&T.fc1_done, 0, &T.abort_flag)) *P.status = 9;
          local_ok = true;
        }
        for (int gg = 0; gg <= g; ++gg) {
          if (passed[gg]) continue;
          bool ok = false;
          for (uint32_t it = 0; it < (1u << 24); ++it) {
            if (ld_acquire_gpu_u64(P.gates + gg) - T.gate0[gg] >= (unsigned long long)V) { ok = true; break; }
            if (T.abort_flag) break;
          }
          if (!ok) { T.abort_flag = 1; *P.status = 3; }
          passed[gg] = true;
          fence_proxy_async();   // the slabs were written through the generic proxy and are read by bulk copies
        }
        flush();
      };
      auto peek_gate = [&](int g) {   // one look, no waiting: gates usually opened long before the tile that needs them is issued
        if (!local_ok && mbar_test_wait(&T.fc1_done, 0)) local_ok = true;
        for (int gg = 0; gg <= g && !passed[gg]; ++gg)
          if (ld_acquire_gpu_u64(P.gates + gg) - T.gate0[gg] >= (unsigned long long)V) { passed[gg] = true; fence_proxy_async(); }
          else break;
        flush();
      };
      int slot = 0, use = 0, mine = pw == 0 ? 0 : kTcProducers - pw;   // `mine` counts down to this producer's next tile
      auto acquire = [&](int gate) {   // the ring slot of the current position, free of its previous occupant
        if (use >= 1) {
          if (gate >= 0) open_gate(gate);   // that occupant may be an FC2 tile still waiting for its activations
          if (!mbar_wait(&T.empty[slot], (use - 1) & 1, &T.abort_flag)) *P.status = 2;
        }
      };
      auto advance = [&]() {
        if (++slot == NS) { slot = 0; ++use; }
        mine = mine == 0 ? kTcProducers - 1 : mine - 1;
      };
      // ---- FC1 tiles: units v, v + V, ... x KB1 boxes; the KB1 records of a unit are contiguous
      for (int t = 0, j = 0; t < nu1; ++t) {
        const int q = v + t * V, u = q / CB1, cb = q - u * CB1;
        const uint8_t* src = P.w1t + ((long long)T.experts[u] * CB1 + cb) * KB1 * kTcStage;
        for (int kb = 0; kb < KB1; ++kb, ++j) {
          if (mine == 0) {
            acquire(-1);
            TC_TRACE(j, 0);
            mbar_expect_tx(&T.full[slot], kTcStage);
            bulk_load_hint(ring + slot * kTcStage, src + (long long)kb * kTcStage, kTcStage, &T.full[slot], pol);
          }
          advance();
        }
      }
      // ---- FC2 tiles: items (u, kb) = r2, r2 + W2, ... of output block nb2; weights (expert of u, nb2, kb), slab (u, kb)
      {
        int u = r2 / KB2, kb = r2 % KB2;
        for (int j = 0; j < n2; ++j) {
          const int g = u < uA ? 0 : 1;
          const int prev_g = j >= NS ? slot_g[slot] : -1;   // gate of the FC2 tile that holds this slot now, if any
          slot_g[slot] = g;
          if (mine == 0) {
            acquire(prev_g);
            TC_TRACE(n1 + j, 0);
            mbar_expect_tx(&T.full[slot], kTcStage + kSlab);
            bulk_load_hint(ring + slot * kTcStage, P.w2t + (((long long)T.experts[u] * NB2 + nb2) * KB2 + kb) * kTcStage, kTcStage, &T.full[slot], pol);
            peek_gate(g);
            if (local_ok && passed[g]) load_slab(slot, u * KB2 + kb);
            else { pend_slot[npend & 15] = slot; pend_idx[npend & 15] = u * KB2 + kb; pend_g[npend & 15] = g; ++npend; }
          }
          kb += dK2, u += dU2;
          if (kb >= KB2) { kb -= KB2; ++u; }
          advance();
        }
      }
      if (pend_head < npend) open_gate(1);
      if (pw == 0) {
        // The kernel after this one in the stream, if it was launched programmatically (the activation expansion of the
        // next layer call is), may be scheduled once every worker has seen gate B open: its blocks start as SMs free up
        // and wait for this grid's completion before they touch any data. Not earlier: a next call on the same workspace
        // reads the gate words at its entry, and they are final only when the last gate of this launch has opened.
        open_gate(1);
        grid_launch_dependents();
      }
#ifdef B200_TIMERS
      if (P.debug && pw == 0) P.debug[v * 16 + 9] = clock64() - tm_begin;
#endif
    }
    __syncwarp();
  } else if (warp >= 4 && warp < 8) {
    // ============================================================== scale warps: one per TMEM lane quadrant
    // The E4M3 scale tiles of a landed stage go shared memory -> registers -> TMEM (tcgen05.st): lane l of every quadrant
    // holds row l of each 512-byte tile (16 bytes = 4 columns). Four warps in parallel replace the 4-8 tcgen05.cp per
    // tile that a single thread would have to issue one after the other.
    const uint32_t lane_base = (uint32_t)((warp - 4) * 32) << 16;
    const uint32_t ring_u = smem_u32(ring) + 16384 + lane * 16, region_u = smem_u32(region);
    const uint32_t xsf_u = smem_u32(xb_sf) + lane * 16;
    int si = 0;
    uint32_t ph = 0;
    auto put = [&](uint32_t src, uint32_t dst_col, int ntiles) {   // up to four consecutive 512-byte tiles -> 16 columns
      uint32_t r[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        uint4 t4 = make_uint4(0u, 0u, 0u, 0u);
        if (j < ntiles) t4 = lds128(src + j * 512);
        r[4 * j] = t4.x, r[4 * j + 1] = t4.y, r[4 * j + 2] = t4.z, r[4 * j + 3] = t4.w;
      }
      tmem_st_32x32b_x16(dst_col + lane_base, r);
    };
    auto publish_sf = [&]() {
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&T.sfr[si]);
      if (++si == NS) { si = 0; ph ^= 1u; }
    };
    if (n1 > 0 && !mbar_wait(&T.xb_full, 0, &T.abort_flag)) *P.status = 6;
    for (int j = 0, kb = 0; j < n1; ++j) {
      if (!mbar_wait(&T.full[si], ph, &T.abort_flag)) *P.status = 1;
      TC_TRACE(j, 1);
      put(ring_u + si * kTcStage, tm_sfa + 16 * si, 4);
      if (j < KB1) put(xsf_u + kb * 2048, tm_sfb + 16 * kb, min(4, P.KT1 - 4 * kb));   // the x operand's scales: once per K box
      publish_sf();
      TC_TRACE(j, 2);
      if (++kb == KB1) kb = 0;
    }
    for (int j = 0; j < n2; ++j) {
      if (!mbar_wait(&T.full[si], ph, &T.abort_flag)) *P.status = 1;
      TC_TRACE(n1 + j, 1);
      put(ring_u + si * kTcStage, tm_sfa + 16 * si, 4);
      put(region_u + si * kSlab + N * 128 + lane * 16, tm_sfb + 16 * si, 4);
      publish_sf();
      TC_TRACE(n1 + j, 2);
    }
    // The routing tables in the router's padded form, for callers that ask for them: written by these four warps of the
    // last worker (the one with the least FC1 work) once their tiles are through, off every critical path.
    if (blockIdx.x == V - 1 && P.experts_out) {
      grid_dependency_wait();   // the tables of the previous call on this workspace may still be read by its tail
      const int t4 = tid - 128;
      for (int e = t4; e < P.E; e += 128)
        if (T.cnt[e] > 0) { P.experts_out[T.uidx[e] - 1] = e; P.offsets_out[T.uidx[e] - 1] = T.base[e] - T.cnt[e]; }
      for (int u = U + t4; u < P.Umax; u += 128) { P.experts_out[u] = -1; P.offsets_out[u + 1] = T.base[kTcMaxE - 1]; }
      if (t4 == 0) P.offsets_out[U] = T.base[kTcMaxE - 1];
      for (int p = t4; p < npairs; p += 128) {
        const int e = T.ids[p];
        if (e < 0) continue;
        int r = 0;
        for (int q = 0; q < p; ++q) r += T.ids[q] == e;
        P.pairs_out[T.base[e] - T.cnt[e] + r] = p;
      }
    }
  } else if (warp == 8) {
    // ============================================================== MMA issuer: the whole warp stays converged
    // Every lane runs the loop with warp-uniform values and one elected lane issues, so descriptors and TMEM addresses
    // can live in uniform registers (issuing from a single diverged lane costs about twice as many cycles per operation).
    const uint32_t el = elect_one();
    const uint32_t idesc = idesc_mxf4nvf4(128, N);
    const uint64_t desc0 = smem_desc_sw128_kmajor(0);
    const uint32_t ring16 = smem_u32(ring) >> 4, region16 = smem_u32(region) >> 4;
    const int nkt_last1 = P.KT1 - 4 * (KB1 - 1), nkt_last2 = P.KT2 - 4 * (KB2 - 1);
    int si = 0, ab = 0, pieces = 0;
    uint32_t ph = 0;
    uint32_t aph[2] = {0, 0};
    auto issue = [&](uint32_t b16, uint32_t sfb, int nkt, bool fresh) {   // the MMAs of the tile in ring slot si
      if (!mbar_wait(&T.sfr[si], ph, &T.abort_flag)) *P.status = 8;     // scale warps arrive after they saw the stage land
      tc_fence_after();
      const uint64_t ad = desc0 | (uint64_t)(ring16 + si * (kTcStage >> 4)), bd = desc0 | (uint64_t)b16;
      const uint32_t acc = tm_acc + 64 * ab, sfa = tm_sfa + 16 * si;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj)
        if (jj < nkt) umma_mxf4nvf4_p(acc, ad + 2 * jj, bd + 2 * jj, idesc, sfa + 4 * jj, sfb + 4 * jj, (fresh && jj == 0) ? 0u : 1u, el);
      umma_commit_p(&T.empty[si], el);
    };
    auto open_piece = [&]() {   // first tile of a piece: the epilogue must have drained this accumulator buffer
      if (pieces >= 2 && !mbar_wait(&T.acc_empty[ab], aph[ab] ^ 1u, &T.abort_flag)) *P.status = 5;
    };
    auto close_piece = [&]() {
      umma_commit_p(&T.acc_full[ab], el);
      aph[ab] ^= 1u;
      ab ^= 1;
      ++pieces;
    };
    if (n1 > 0) {
      if (!mbar_wait(&T.xb_full, 0, &T.abort_flag)) *P.status = 6;
      tc_fence_after();
    }
    for (int j = 0, kb = 0; j < n1; ++j) {
      if (kb == 0) open_piece();
      issue(region16 + kb * ((N * 128) >> 4), tm_sfb + 16 * kb, kb == KB1 - 1 ? nkt_last1 : 4, kb == 0);
      TC_TRACE(j, 4);
      if (++kb == KB1) { kb = 0; close_piece(); }
      if (++si == NS) { si = 0; ph ^= 1u; }
    }
    if (n1 > 0) umma_commit_p(&T.fc1_done, el);   // the x operand's shared memory and scale columns may be reused from here on
    if (n2 > 0) {   // one piece: all of this worker's items of output block nb2 go into one accumulator
      open_piece();
      for (int j = 0, kb = r2 % KB2; j < n2; ++j) {
        issue(region16 + si * (kSlab >> 4), tm_sfb + 16 * si, kb == KB2 - 1 ? nkt_last2 : 4, j == 0);
        TC_TRACE(n1 + j, 4);
        kb += dK2;
        if (kb >= KB2) kb -= KB2;
        if (++si == NS) { si = 0; ph ^= 1u; }
      }
      close_piece();
    }
#ifdef B200_TIMERS
    if (P.debug && lane == 0) { P.debug[v * 16 + 6] = clock64() - tm_begin; P.debug[v * 16 + 12] = n1 + n2; }
#endif
  } else {
    // ============================================================== epilogue: 4 warps, thread = accumulator row
    const int et = tid;                            // 0..127
    const int quad = warp;                     // TMEM lane quadrant this warp may read
    const int row = quad * 32 + lane;              // accumulator row (MMA M index)
    __shared__ float s_ex[64][17];                 // gate values / activations of one unit: [column][token]
    __shared__ float s_w[16];
    grid_dependency_wait();   // everything before this kernel in the stream is complete and visible from here on
    if (et == 0 && n1 > 0) {
      // the resident B operand of FC1 (x expanded into NVFP4 terms by the kernel launched just before this one) and its
      // scale tiles: one bulk copy
      mbar_expect_tx(&T.xb_full, KB1 * (N * 128) + P.KT1 * 512);
      bulk_load(region, P.xb, KB1 * (N * 128) + P.KT1 * 512, &T.xb_full);
    }
    if (et < N) T.colscale[et] = P.xscale[et];
    // The routing inputs were read at entry, before the wait above, so that the weight stream could start early. If they
    // were still being written then (a producer kernel that lets its successors start before it has written them), the
    // copies used here are stale: say so instead of returning a wrong result silently.
    for (int p = et; p < npairs; p += 128) {
      int e2 = (int)ld_acquire_gpu(reinterpret_cast<const unsigned*>(P.ids) + p);
      if (e2 < 0 || e2 >= P.E) e2 = -1;
      const unsigned w2 = ld_acquire_gpu(reinterpret_cast<const unsigned*>(P.wts) + p);
      if (e2 != T.ids[p] || w2 != __float_as_uint(T.wts[p])) P.status[2] = 1;
    }
    named_bar_sync(1, 128);
    int ab = 0;
    uint32_t aph[2] = {0, 0};
    auto load_terms = [&](float (&val)[16], const float* cs, bool per_column) {   // sum the four term columns of every token
      TC_T0(t0);
      if (!mbar_wait(&T.acc_full[ab], aph[ab], &T.abort_flag)) *P.status = 7;
      TC_ADD(tm_a, t0);
#ifdef B200_TIMERS
      if (tm_d == 0) tm_d = clock64() - tm_begin;   // first accumulator ready
#endif
      tc_fence_after();
      uint32_t r[NB][16];   // all columns in flight before the one wait
#pragma unroll
      for (int c = 0; c < NB; ++c) tmem_ld_32x32b_x16(tm_acc + 64 * ab + ((uint32_t)(quad * 32) << 16) + 16 * c, r[c]);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < NB; ++c) {
#pragma unroll
        for (int tk = 0; tk < 4; ++tk) {
          const int o = per_column ? 16 * c + 4 * tk : 0;
          val[4 * c + tk] = __uint_as_float(r[c][4 * tk]) * cs[o] + __uint_as_float(r[c][4 * tk + 1]) * cs[o + 1] +
                            __uint_as_float(r[c][4 * tk + 2]) * cs[o + 2] + __uint_as_float(r[c][4 * tk + 3]) * cs[o + 3];
        }
      }
#pragma unroll
      for (int i = N / 4; i < 16; ++i) val[i] = 0.f;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&T.acc_empty[ab]);
      aph[ab] ^= 1u;
      ab ^= 1;
    };
    // Sum of the partials of workers vlo..vhi in worker order (a fixed order: bit-identical from call to call). A partial
    // holds N/4 floats per row; kRedBatch workers are loaded at once so that the L2 round trips overlap.
    constexpr int kRedBatch = NB == 4 ? 6 : 12;
    auto reduce = [&](int vlo, int nlive, float (&val)[16]) {
#pragma unroll
      for (int i = 0; i < 16; ++i) val[i] = 0.f;
      for (int p0 = 0; p0 < nlive; p0 += kRedBatch) {
        float4 tmp[kRedBatch][NB];
#pragma unroll
        for (int b = 0; b < kRedBatch; ++b) {
          const bool live = p0 + b < nlive;
          const float* src = P.scratch + ((long long)((vlo + (live ? p0 + b : 0)) * 2) * 128 + et) * 16;
#pragma unroll
          for (int i = 0; i < NB; ++i) tmp[b][i] = live ? __ldcg(reinterpret_cast<const float4*>(src) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int b = 0; b < kRedBatch; ++b)
          if (p0 + b < nlive) {
#pragma unroll
            for (int i = 0; i < NB; ++i) { val[4 * i] += tmp[b][i].x; val[4 * i + 1] += tmp[b][i].y; val[4 * i + 2] += tmp[b][i].z; val[4 * i + 3] += tmp[b][i].w; }
          }
      }
    };
    // publish this worker's partial of its output block and learn whether it arrived last of the `nlive` holders
    auto publish = [&](const float (&val)[16], unsigned* counter, int nlive) -> bool {
      float* mine = P.scratch + ((long long)(v * 2) * 128 + et) * 16;
#pragma unroll
      for (int i = 0; i < NB; ++i) *reinterpret_cast<float4*>(mine + 4 * i) = make_float4(val[4 * i], val[4 * i + 1], val[4 * i + 2], val[4 * i + 3]);
      named_bar_sync(1, 128);
      if (et == 0) {
        const unsigned old = atom_add_acq_rel_gpu(counter, 1u);   // releases the partial (barrier above), acquires the others'
        const int last = old + 1u == (unsigned)nlive;
        if (last) *counter = 0;   // nobody touches the counter again before the next launch
        T.last_flag = last;
      }
      named_bar_sync(1, 128);
      return T.last_flag != 0;   // the next write of last_flag is behind at least one more barrier of these 128 threads
    };
    // arrive at gate g of FC1: everything this worker wrote for the experts of the gate's group is visible to the TMA
    // loads of every worker that sees the gate open (the producers are the only waiters)
    auto arrive_gate = [&](int g) {
      fence_proxy_async();
      named_bar_sync(1, 128);
      if (et == 0) red_add_release_gpu_u64(P.gates + g, 1ull);   // nothing to wait for: the gate is open when V have arrived
    };

    // ---- FC1 pieces
    {
      if (use_gate_a && nuA == 0) arrive_gate(0);
      if (nu1 == 0) arrive_gate(1);
      for (int t = 0; t < nu1; ++t) {
        const int q = v + t * V, u = q / CB1, cb = q - u * CB1;   // a whole unit: K boxes 0..KB1-1 of (expert u, block cb)
        const int e = T.experts[u];
        float val[16];
        load_terms(val, T.colscale, true);
        TC_T0(tfix);
        {
          // rows 0..63 hold the up columns 64cb.., rows 64..127 the gate columns: exchange through shared memory.
          // s_w[tk]: routing weight of token tk on this expert folded with alpha2 (relative to the layer's largest), 0 when
          // the token is not routed here - only routed tokens cost any arithmetic below.
          const float alpha = T.a1[u];
          if (et < 16) {
            float wsum = 0.f;
            if (et < P.M)
              for (int sidx = 0; sidx < P.top_k; ++sidx)
                if (T.ids[et * P.top_k + sidx] == e) wsum += T.wts[et * P.top_k + sidx];
            s_w[et] = wsum * T.a2n[u];
          }
          if (row >= 64) {
#pragma unroll
            for (int tk = 0; tk < 16; ++tk) s_ex[row - 64][tk] = val[tk] * alpha;
          }
          named_bar_sync(1, 128);
          if (row < 64) {
#pragma unroll
            for (int tk = 0; tk < 16; ++tk) {
              const float wf = s_w[tk];
              s_ex[row][tk] = wf != 0.f ? tc_silu_mul(s_ex[row][tk], val[tk] * alpha) * wf : 0.f;   // only this thread reads that gate value
            }
          }
          named_bar_sync(1, 128);
          // re-expand: thread (token, 16-column block) -> four NVFP4 terms of the FC2 operand; a token that is not routed
          // here only gets zero scale bytes (a zero scale silences whatever codes the row holds). (Spreading a block over
          // four lanes - expand_block16_quad - was measured: no gain at any batch size, the expansion is off the critical path.)
          if (et < N) {
            const int tk = et >> 2, blk = et & 3;
            uint8_t* slab = P.aslab + ((long long)u * KB2 + (cb >> 2)) * kSlab;   // slab of K box cb/4
            uint8_t* sfp = slab + N * 128 + (cb & 3) * 512 + blk;
            const int chunk = 2 * (cb & 3) + (blk >> 1);                        // 16-byte chunk of the row's 128 bytes
            if (s_w[tk] != 0.f) {
              float r[16];
#pragma unroll
              for (int i = 0; i < 16; ++i) r[i] = s_ex[blk * 16 + i][tk];
              uint2 codes[kTerms];
              uint8_t sf[kTerms];
              if (expand_block16(r, P.act_g1, codes, sf)) P.status[1] = 1;   // beyond the range of the fixed activation scale
#pragma unroll
              for (int t = 0; t < kTerms; ++t) {
                const int n = tk * kTerms + t;
                *reinterpret_cast<uint2*>(slab + n * 128 + ((chunk ^ (n & 7)) << 4) + (blk & 1) * 8) = codes[t];
                sfp[(n & 31) * 16 + (n >> 5) * 4] = sf[t];
              }
            } else {
#pragma unroll
              for (int t = 0; t < kTerms; ++t) {
                const int n = tk * kTerms + t;
                sfp[(n & 31) * 16 + (n >> 5) * 4] = 0;
              }
            }
          }
          named_bar_sync(1, 128);
        }
        TC_ADD(tm_b, tfix);
        if (use_gate_a && t == nuA - 1) arrive_gate(0);
        if (t == nu1 - 1) arrive_gate(1);
      }
#ifdef B200_TIMERS
      tm_c = clock64() - tm_begin;
#endif
    }
    // ---- FC2: this worker's items of output block nb2, summed over experts and K boxes inside the tensor core
    if (n2 > 0) {
      float cs[kTerms];   // 1 / g_t of the activation terms, times the alpha2 the operand was normalised by
      {
        float g = P.act_g1;
        const float a2ref = P.alpha2_ref[0];
#pragma unroll
        for (int t = 0; t < kTerms; ++t) { cs[t] = a2ref / g; g *= 6.0f; }
      }
      float val[16];
      load_terms(val, cs, false);
      if (publish(val, P.cnt2 + nb2, live2)) {
        reduce(vlo2, live2, val);
#pragma unroll
        for (int tk = 0; tk < 16; ++tk)
          if (tk < P.M) P.out[(long long)tk * P.H + 128 * nb2 + row] = __float2bfloat16_rn(val[tk]);
      }
    } else if (I2 == 0 && r2 == 0) {   // every slot of the batch is empty: the layer's output is zero
      for (int tk = 0; tk < P.M; ++tk) P.out[(long long)tk * P.H + 128 * nb2 + row] = __float2bfloat16_rn(0.f);
    }
#ifdef B200_TIMERS
    if (P.debug && et == 0) { P.debug[v * 16 + 0] = tm_a; P.debug[v * 16 + 1] = tm_b; P.debug[v * 16 + 2] = tm_c; P.debug[v * 16 + 3] = tm_d; P.debug[v * 16 + 7] = clock64() - tm_begin; }
#endif
  }
  tc_fence_before();
  __syncthreads();
#ifdef B200_TIMERS
  if (tid == 0 && P.debug) { unsigned long long g; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g)); P.debug[blockIdx.x * 16 + 14] = (long long)g; }
#endif
  if (warp == 8) tmem_dealloc(tmem, 512);
  if (T.abort_flag)
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
}

}  // namespace b200

using namespace b200;

int b200_decode_tc_smem_bytes(int NS, int region_bytes) { return 1024 + NS * kTcStage + region_bytes + (int)sizeof(TcTables); }

static bool pdl_chain_enabled() {   // B200MOE_PDL_CHAIN=0: launch the expansion kernel as an ordinary stream-ordered kernel
  static const bool on = [] { const char* c = getenv("B200MOE_PDL_CHAIN"); return !(c && c[0] == '0'); }();
  return on;
}

int b200_expand_x_launch(const void* x, int M, int H, int N, int KB1, void* xb, float* colscale, bool chained, cudaStream_t st) {
  // programmatic launch: the blocks may be scheduled while the previous kernel of the stream drains (if that kernel
  // allows it, as this library's layer kernel does); griddepcontrol.wait at their top keeps stream order for all data
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(N / kTerms), cfg.blockDim = dim3(128), cfg.dynamicSmemBytes = 0, cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = chained && pdl_chain_enabled() ? 1 : 0;
  const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
  uint8_t* xbp = (uint8_t*)xb;
  void* args[] = {(void*)&xp, (void*)&M, (void*)&H, (void*)&N, (void*)&KB1, (void*)&xbp, (void*)&colscale};
  B200_CUDA_TRY(cudaLaunchKernelExC(&cfg, (const void*)k_expand_x, args));
  return B200MOE_OK;
}

// q u8 [E, rows, row_bytes], sf = 128x4-swizzled scales per expert -> tile records (see k_pack_tiles)
int b200_pack_tiles_launch(const void* q, const void* sf, void* out, int E, int rows_per_expert, int row_bytes, int blocks, int KB, int KT,
                           int fc1, int I, long long sf_stride, cudaStream_t st) {
  const long long total = (long long)E * blocks * KB * 1152;
  long long g = (total + 255) / 256;
  if (g > 148 * 32) g = 148 * 32;
  k_pack_tiles<<<(int)g, 256, 0, st>>>((const uint8_t*)q, (const uint8_t*)sf, (uint8_t*)out, E, rows_per_expert, row_bytes, blocks, KB, KT, fc1,
                                       I, sf_stride);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

int b200_decode_tc_launch(const DecodeTcParams& p, int grid, int smem_bytes, bool chained, cudaStream_t st) {
  void* args[] = {(void*)&p};
  const void* fn = p.M <= 4 ? (const void*)k_moe_decode_tc<1> : p.M <= 8 ? (const void*)k_moe_decode_tc<2> : (const void*)k_moe_decode_tc<4>;
  static thread_local int configured[3] = {0, 0, 0};
  const int which = p.M <= 4 ? 0 : p.M <= 8 ? 1 : 2;
  if (configured[which] < smem_bytes) {
    B200_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    configured[which] = smem_bytes;
  }
  // programmatic dependent launch: this kernel's prologue and weight prefetch overlap the activation-expansion kernel
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid), cfg.blockDim = dim3(kTcThreads), cfg.dynamicSmemBytes = (size_t)smem_bytes, cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = chained ? 1 : 0;
  B200_CUDA_TRY(cudaLaunchKernelExC(&cfg, fn, args));
  return B200MOE_OK;
}
