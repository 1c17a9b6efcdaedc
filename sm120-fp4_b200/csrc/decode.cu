// The decode-regime (M <= 16 tokens) W4A16 MoE layer as ONE persistent kernel: routing, FC1 (+SiLU*mul) and FC2
// (+ top-k weighted combine). It replaces the reference's three launches k_route / k_fc1* / k_fc2* of
// sm120fp4/kernels/{moe_w4a16,fc1_w4a16,fc1_mma,fc2_w4a16,fc2_mma_pf}.py; the arithmetic contract is theirs
// (FP4 code x E4M3 block scale, fp32 accumulation, alpha applied in fp32, __expf SiLU, one rounding of the output).
//
// Structure (B200-first, memory-bound):
//  * one CTA per SM; warps 0-3 and 4-7 are two consumer groups ("workers"), warps 8 and 9 their TMA producers.
//  * the work is a flat list of weight tiles: FC1 tile = 64 up rows + 64 gate rows x 256 K-codes (two 8 KB TMA boxes,
//    128B swizzle) + their 128x4 scale runs; FC2 tile = 128 output rows x 256 K-codes + scale run + the activation slab
//    of that expert / K-box. Every worker owns a contiguous, equal share of the flat list (stream-K), so any number of
//    touched experts balances over the 2 x #SM workers.
//  * tiles land in a ring of shared-memory stages guarded by full/empty mbarriers; the producer runs ahead of the math by
//    the ring depth and, across the FC1->FC2 dependency, prefetches FC2 weight tiles before the grid-wide barrier opens.
//  * math: codes -> f16 with cvt.rn.f16x2.e2m1x2, times the E4M3 scale (exact in f16), mma.sync m16n8k16 f16 with fp32
//    accumulators, tokens as the N dimension ("global token columns": column j is token j for every expert, so partial
//    sums of different experts add in registers and the routing weight is applied per expert in fp32).
//  * a tile range that cuts a unit writes its partial sums to an L2-resident scratch; the last arriver (atomic counter)
//    adds the pieces in worker order, so the result is bit-identical from call to call.
#include "common.cuh"
#include "ptx.cuh"
#include "decode_params.h"

namespace b200 {

constexpr int kConsumerWarps = 8;
constexpr int kGroupThreads = 128;
constexpr int kThreads = (kConsumerWarps + 2) * 32;   // + one TMA producer warp per consumer group
constexpr int kSlotBytes = 20480;      // 16 KB codes + 4 KB scales
constexpr int kCodesBytes = 16384;
constexpr int kMaxE = 256, kMaxP = 256;
constexpr int kMaxWorkers = 512;       // 2 x SM count

enum { ST_OK = 0, ST_TIMEOUT_FULL = 1, ST_TIMEOUT_EMPTY = 2, ST_TIMEOUT_GRID = 3, ST_BAD_ID = 4 };

struct Tables {
  int ids[kMaxP];
  float wts[kMaxP];
  int cnt[kMaxE];      // pairs per expert
  int base[kMaxE];     // inclusive scan of cnt
  int uidx[kMaxE];     // inclusive scan of touched flags
  int experts[kMaxE];  // touched experts ascending
  unsigned omask[kMaxE];  // per touched expert: bit n set when a token of octet n (tokens 8n..8n+7) is routed to it
  int sb1[kMaxWorkers + 1];   // first FC1 tile of every worker (stream-K shares); sb1[V] = T1
  int sb2[kMaxWorkers + 1];   // same for FC2
  int U;
  unsigned gen0;       // grid-barrier generation at kernel start
  volatile int abort_flag;
  int last_flag[2];
  uint64_t full[8];
  uint64_t empty[8];
};

__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.0f + __expf(-gate)) * up; }

// Owner of flat tile f when worker v owns [v*T/V, (v+1)*T/V): ceil((f+1)*V/T) - 1. Products stay below 2^31 (host check).
__device__ __forceinline__ int worker_of(int f, int T, int V) { return (int)(((unsigned)(f + 1) * (unsigned)V - 1u) / (unsigned)T); }

#ifdef B200_TIMERS
#define TIMER_START(var) long long var = clock64()
#define TIMER_ADD(acc, var) acc += clock64() - var
#else
#define TIMER_START(var)
#define TIMER_ADD(acc, var)
#endif

// One weight tile through the tensor cores for one warp: two 16-row blocks (rb) x 256 K-codes, NB8 token octets.
// acc[parity][rb][n][4]: even and odd MMAs of a K run use separate accumulators to halve the dependent chain.
template <int NB8>
__device__ __forceinline__ void mma_tile(uint32_t codes, int row0, int row1, uint32_t sc0, int rt0, uint32_t sc1, int rt1,
                                         bool kt_valid, uint32_t bfrag, int lane, unsigned octets, float (&acc)[2][2][NB8][4]) {
  const int g = lane >> 2, t = lane & 3;
  uint32_t sfw[2][2];
  {
    const int r00 = rt0 + g, r01 = rt0 + g + 8, r10 = rt1 + g, r11 = rt1 + g + 8;
    sfw[0][0] = kt_valid ? lds32(sc0 + t * 512 + (r00 & 31) * 16 + (r00 >> 5) * 4) : 0u;
    sfw[0][1] = kt_valid ? lds32(sc0 + t * 512 + (r01 & 31) * 16 + (r01 >> 5) * 4) : 0u;
    sfw[1][0] = kt_valid ? lds32(sc1 + t * 512 + (r10 & 31) * 16 + (r10 >> 5) * 4) : 0u;
    sfw[1][1] = kt_valid ? lds32(sc1 + t * 512 + (r11 & 31) * 16 + (r11 >> 5) * 4) : 0u;
  }
#pragma unroll 1
  for (int h = 0; h < 2; ++h) {
    uint4 bq[4][NB8];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj)
#pragma unroll
      for (int n = 0; n < NB8; ++n)
        if (NB8 == 1 || ((octets >> n) & 1u)) bq[jj][n] = lds128(bfrag + ((((h * 4 + jj) * NB8 + n) * 32 + lane) << 4));
#pragma unroll
    for (int rb = 0; rb < 2; ++rb) {
      const int ra = (rb == 0 ? row0 : row1) + g;   // stage row of fragment row g; fragment row g+8 is ra+8
      const uint32_t chunk = (uint32_t)(((2 * t + h) ^ (ra & 7)) << 4);
      const uint4 qa = lds128(codes + ra * 128 + chunk);
      const uint4 qb = lds128(codes + (ra + 8) * 128 + chunk);
      const uint32_t sa = cvt_e4m3x2_f16x2(sfw[rb][0] >> (16 * h));
      const uint32_t sb = cvt_e4m3x2_f16x2(sfw[rb][1] >> (16 * h));
      const uint32_t sa_lo = prmt(sa, sa, 0x1010), sa_hi = prmt(sa, sa, 0x3232);
      const uint32_t sb_lo = prmt(sb, sb, 0x1010), sb_hi = prmt(sb, sb, 0x3232);
      const uint32_t wa[4] = {qa.x, qa.y, qa.z, qa.w}, wb[4] = {qb.x, qb.y, qb.z, qb.w};
#pragma unroll
      for (int wd = 0; wd < 4; ++wd) {
        uint32_t da[4], db[4];
        cvt_e2m1x8_f16x2(wa[wd], da);
        cvt_e2m1x8_f16x2(wb[wd], db);
        const uint32_t s_a = wd < 2 ? sa_lo : sa_hi, s_b = wd < 2 ? sb_lo : sb_hi;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          da[i] = hmul2_u32(da[i], s_a);
          db[i] = hmul2_u32(db[i], s_b);
        }
#pragma unroll
        for (int n = 0; n < NB8; ++n)
          if (NB8 == 1 || ((octets >> n) & 1u)) {   // warp-uniform: skip a token octet no token of which is routed here
            mma_f16_16816(acc[0][rb][n], da[0], db[0], da[1], db[1], bq[wd][n].x, bq[wd][n].y);
            mma_f16_16816(acc[1][rb][n], da[2], db[2], da[3], db[3], bq[wd][n].z, bq[wd][n].w);
          }
      }
    }
  }
}

// half index inside the fragment-ordered activation buffer of one expert slot, for K index k and token tok
template <int NB8>
__device__ __forceinline__ int frag_index(int k, int tok) {
  const int kb = k >> 8, tq = (k & 255) >> 6, h = (k & 63) >> 5, jj = (k & 31) >> 3;
  const int lane = ((tok & 7) << 2) | tq;
  return kb * (NB8 * 2048) + ((((h * 4 + jj) * NB8 + (tok >> 3)) * 32 + lane) << 3) + (k & 7);
}

// Sum the partial results of the workers [vlo, vhi] that own a piece of the unit starting at flat tile `first`, in worker
// order (fixed summation order), four pieces' loads in flight at a time. v[] has 8*NB8 floats per thread.
template <int NB8>
__device__ __forceinline__ void reduce_pieces(const float* __restrict__ scratch, const int* sb, int first, int vlo, int vhi,
                                              int gtid, float (&v)[8 * NB8]) {
#pragma unroll
  for (int i = 0; i < 8 * NB8; ++i) v[i] = 0.f;
  for (int p0 = vlo; p0 <= vhi; p0 += 4) {
    float4 tmp[4][2 * NB8];
    bool live[4];
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int pv = p0 + b;
      live[b] = pv <= vhi && sb[pv + 1] > sb[pv];
      const int pslot = (live[b] && sb[pv] < first) ? 1 : 0;   // a piece that starts its worker's share sits in slot 0
      const float* src = scratch + ((long long)((live[b] ? pv : vlo) * 2 + pslot) * kGroupThreads + gtid) * 16;
#pragma unroll
      for (int i = 0; i < 2 * NB8; ++i)
        tmp[b][i] = live[b] ? __ldcg(reinterpret_cast<const float4*>(src) + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int b = 0; b < 4; ++b)
      if (live[b]) {
#pragma unroll
        for (int i = 0; i < 2 * NB8; ++i) {
          v[4 * i] += tmp[b][i].x, v[4 * i + 1] += tmp[b][i].y, v[4 * i + 2] += tmp[b][i].z, v[4 * i + 3] += tmp[b][i].w;
        }
      }
  }
}

template <int NB8>
__global__ void __launch_bounds__(kThreads, 1) k_moe_decode(const __grid_constant__ DecodeParams P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int NS = P.NS;                          // ring stages (even); worker g uses slots 2*i+g
  uint8_t* ring = smem;
  uint8_t* region = smem + NS * kSlotBytes;     // FC1: x in fragment order (f16); FC2: activation slabs per ring slot
  Tables& T = *reinterpret_cast<Tables*>(region + P.region_bytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int npairs = P.M * P.top_k;
  const int V = 2 * gridDim.x;

  // ---------------------------------------------------------------- prologue: barriers + routing tables (every CTA)
  if (tid == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(&T.full[s], 1);
      mbar_init(&T.empty[s], 4);
    }
    T.abort_flag = 0;
    T.last_flag[0] = T.last_flag[1] = 0;
    // read before any group of this CTA can arrive, so the generation cannot have advanced yet
    T.gen0 = ld_acquire_gpu(P.gridbar + 1);
    fence_mbar_init();
  }
  if (tid < kMaxE) T.cnt[tid] = 0;
  __syncthreads();
  for (int p = tid; p < npairs; p += kThreads) {
    int e = P.ids[p];   // a negative id marks an empty slot (expert-parallel shards mask the experts they do not own)
    if (e >= P.E) { *P.status = ST_BAD_ID; e = -1; }
    if (e < 0) e = -1;
    T.ids[p] = e;
    T.wts[p] = P.wts[p];
    if (e >= 0) atomicAdd(&T.cnt[e], 1);
  }
  __syncthreads();
  if (warp == 0) {   // inclusive scans over kMaxE entries, 8 per lane
    int c[8], f[8], sc = 0, sf = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      c[i] = T.cnt[lane * 8 + i];
      f[i] = c[i] > 0;
      sc += c[i];
      sf += f[i];
    }
    int ic = sc, iff = sf;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, ic, o), b = __shfl_up_sync(0xffffffffu, iff, o);
      if (lane >= o) { ic += a; iff += b; }
    }
    int rc = ic - sc, rf = iff - sf;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      rc += c[i];
      rf += f[i];
      T.base[lane * 8 + i] = rc;
      T.uidx[lane * 8 + i] = rf;
    }
    if (lane == 31) T.U = iff;
  }
  __syncthreads();
  const int U = T.U;
  const bool do1 = (P.phases & 1) != 0, do2 = (P.phases & 2) != 0;
  const int KB1 = P.KB1, KB2 = P.KB2, CB1 = P.CB1, NB2 = P.NB2;
  const int T1 = do1 ? U * CB1 * KB1 : 0;
  const int T2 = do2 ? NB2 * U * KB2 : 0;
  if (tid < kMaxE && T.cnt[tid] > 0) {
    T.experts[T.uidx[tid] - 1] = tid;
    unsigned m = 0;
    for (int tok = 0; tok < P.M; ++tok)
      for (int sidx = 0; sidx < P.top_k; ++sidx)
        if (T.ids[tok * P.top_k + sidx] == tid) m |= 1u << (tok >> 3);
    T.omask[T.uidx[tid] - 1] = m;
  }
  for (int v = tid; v <= V; v += kThreads) {   // stream-K shares: worker v owns tiles [sb[v], sb[v+1])
    T.sb1[v] = (int)(((unsigned)v * (unsigned)T1) / (unsigned)V);
    T.sb2[v] = (int)(((unsigned)v * (unsigned)T2) / (unsigned)V);
  }
  __syncthreads();

  if (blockIdx.x == 0 && P.experts_out) {   // the routing tables in the reference's padded form
    const int Umax = P.Umax;
    for (int e = tid; e < P.E; e += kThreads)
      if (T.cnt[e] > 0) {
        P.experts_out[T.uidx[e] - 1] = e;
        P.offsets_out[T.uidx[e] - 1] = T.base[e] - T.cnt[e];
      }
    for (int u = U + tid; u < Umax; u += kThreads) {
      P.experts_out[u] = -1;
      P.offsets_out[u + 1] = T.base[kMaxE - 1];
    }
    if (tid == 0) P.offsets_out[U] = T.base[kMaxE - 1];   // number of routed pairs (= npairs when no slot is empty)
    for (int p = tid; p < npairs; p += kThreads) {
      const int e = T.ids[p];
      if (e < 0) continue;
      int r = 0;
      for (int q = 0; q < p; ++q) r += T.ids[q] == e;
      P.pairs_out[T.base[e] - T.cnt[e] + r] = p;
    }
  }

  const int slab_bytes = NB8 * 4096;
  const int per = NS / 2;
#ifdef B200_TIMERS
  long long tm_wait = 0, tm_mma = 0, tm_fix = 0, tm_pwait = 0, tm_pgrid = 0;
  const long long tm_begin = clock64();
#endif

  if (warp >= kConsumerWarps) {
    // ============================================================== producers: warp 8 feeds group 0, warp 9 group 1
    if (lane == 0) {
      const int grp = warp - kConsumerWarps;
      const int v = 2 * blockIdx.x + grp;
      prefetch_tensormap(&P.tm1);
      prefetch_tensormap(&P.tm2);
      const uint64_t pol = policy_evict_first();
      const unsigned gen0 = T.gen0;
      bool passed = !do1;            // without an FC1 phase the activations are already in place
      const int n1 = T.sb1[v + 1] - T.sb1[v], n2 = T.sb2[v + 1] - T.sb2[v];
      int pend_slot[4];
      const uint8_t* pend_src[4];
      int npend = 0;
      auto wait_grid = [&]() {
        if (passed) return;
        TIMER_START(t0);
        bool ok = false;
        for (uint32_t it = 0; it < (1u << 24); ++it) {
          if (ld_acquire_gpu(P.gridbar + 1) != gen0) { ok = true; break; }
          if (T.abort_flag) break;
          __nanosleep(64);
        }
        if (!ok) { T.abort_flag = 1; *P.status = ST_TIMEOUT_GRID; }
        fence_proxy_async();
        for (int i = 0; i < npend; ++i)
          bulk_load(region + pend_slot[i] * slab_bytes, pend_src[i], slab_bytes, &T.full[pend_slot[i]]);
        npend = 0;
        passed = true;
        TIMER_ADD(tm_pgrid, t0);
      };
      int si = 0;           // ring position of this group (0..per-1)
      uint32_t ph = 0;      // parity of the current pass over the ring
      int j = 0;            // tiles issued
      auto claim_slot = [&](bool prev_was_fc2_pending) -> int {
        const int slot = 2 * si + grp;
        if (j >= per) {
          if (prev_was_fc2_pending) wait_grid();   // the previous occupant still waits for its activations: open the gate first
          TIMER_START(t0);
          if (!mbar_wait(&T.empty[slot], ph ^ 1u, &T.abort_flag)) *P.status = ST_TIMEOUT_EMPTY;
          TIMER_ADD(tm_pwait, t0);
        }
        return slot;
      };
      auto advance = [&]() {
        ++j;
        if (++si == per) { si = 0; ph ^= 1u; }
      };
      // ---- FC1 tiles of this worker, in flat order (expert slot u, column block cb, K box kb)
      if (n1 > 0) {
        const int f0 = T.sb1[v];
        int kb = f0 % KB1, q = f0 / KB1, cb = q % CB1, u = q / CB1;
        for (int i = 0; i < n1; ++i) {
          const int slot = claim_slot(false);
          uint8_t* st = ring + slot * kSlotBytes;
          const int e = T.experts[u];
          const int nkt = min(4, P.KT1 - 4 * kb);
          const int up_row = 64 * cb, gate_row = P.I + 64 * cb;
          mbar_expect_tx(&T.full[slot], kCodesBytes + 2 * nkt * 512);
          tma_load_2d_hint(st, &P.tm1, 128 * kb, e * 2 * P.I + up_row, &T.full[slot], pol);
          tma_load_2d_hint(st + 8192, &P.tm1, 128 * kb, e * 2 * P.I + gate_row, &T.full[slot], pol);
          const uint8_t* sbase = P.s1 + (long long)e * P.s1_expert_stride;
          bulk_load_hint(st + kCodesBytes, sbase + ((long long)(up_row >> 7) * P.KT1 + 4 * kb) * 512, nkt * 512, &T.full[slot], pol);
          bulk_load_hint(st + kCodesBytes + 2048, sbase + ((long long)(gate_row >> 7) * P.KT1 + 4 * kb) * 512, nkt * 512, &T.full[slot], pol);
          advance();
          if (++kb == KB1) { kb = 0; if (++cb == CB1) { cb = 0; ++u; } }
        }
      }
      // ---- FC2 tiles, in flat order (output block nb, expert slot u, K box kb); weights run ahead of the grid barrier
      if (n2 > 0) {
        const int f0 = T.sb2[v];
        int kb = f0 % KB2, q = f0 / KB2, u = q % U, nb = q / U;
        for (int i = 0; i < n2; ++i) {
          const int slot = claim_slot(!passed && (j - per) >= n1);
          uint8_t* st = ring + slot * kSlotBytes;
          const int e = T.experts[u];
          const int nkt = min(4, P.KT2 - 4 * kb);
          mbar_expect_tx(&T.full[slot], kCodesBytes + nkt * 512 + slab_bytes);
          tma_load_2d_hint(st, &P.tm2, 128 * kb, e * P.H + 128 * nb, &T.full[slot], pol);
          bulk_load_hint(st + kCodesBytes, P.s2 + (long long)e * P.s2_expert_stride + ((long long)nb * P.KT2 + 4 * kb) * 512,
                         nkt * 512, &T.full[slot], pol);
          const uint8_t* src = reinterpret_cast<const uint8_t*>(P.actfrag) + ((long long)u * KB2 + kb) * slab_bytes;
          if (passed) bulk_load(region + slot * slab_bytes, src, slab_bytes, &T.full[slot]);
          else { pend_slot[npend] = slot; pend_src[npend] = src; ++npend; }
          advance();
          if (++kb == KB2) { kb = 0; if (++u == U) { u = 0; ++nb; } }
        }
      }
      if (npend > 0) wait_grid();
#ifdef B200_TIMERS
      if (P.debug) { P.debug[v * 8 + 4] = tm_pwait; P.debug[v * 8 + 5] = tm_pgrid; P.debug[v * 8 + 6] = clock64() - tm_begin; }
#endif
    }
    __syncwarp();
  } else {
    // ============================================================== consumers: two groups of four warps
    const int grp = warp >> 2, w = warp & 3;
    const int v = 2 * blockIdx.x + grp;
    const int gtid = tid & (kGroupThreads - 1);
    const int g = lane >> 2, t = lane & 3;
    const uint32_t ring_a = smem_u32(ring), region_a = smem_u32(region);
    int si = 0;
    uint32_t ph = 0;

    if (do1) {
      // ---- stage x as f16 in fragment order (all 256 consumer threads), zero beyond M tokens / H columns
      const int chunks_per_tok = KB1 * 32;   // 16-byte chunks (8 values) per token over the padded K
      for (int i = tid; i < 8 * NB8 * chunks_per_tok; i += kConsumerWarps * 32) {
        const int tok = i / chunks_per_tok, c8 = i % chunks_per_tok, k = c8 * 8;
        uint4 outv = make_uint4(0u, 0u, 0u, 0u);
        if (tok < P.M && k < P.H) {
          const uint4 raw = *reinterpret_cast<const uint4*>(P.x + (long long)tok * P.H + k);
          const uint32_t wsrc[4] = {raw.x, raw.y, raw.z, raw.w};
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float lo = __uint_as_float(wsrc[q] << 16), hi = __uint_as_float(wsrc[q] & 0xffff0000u);
            const __half2 hv = __floats2half2_rn(fminf(fmaxf(lo, -65504.f), 65504.f), fminf(fmaxf(hi, -65504.f), 65504.f));
            o[q] = *reinterpret_cast<const uint32_t*>(&hv);
          }
          outv = make_uint4(o[0], o[1], o[2], o[3]);
        }
        *reinterpret_cast<uint4*>(region + frag_index<NB8>(k, tok) * 2) = outv;
      }
      named_bar_sync(3, kConsumerWarps * 32);

      // ---- FC1 pieces of this worker
      const int fs = T.sb1[v], fe = T.sb1[v + 1];
      int f = fs;
      while (f < fe) {
        const int q = f / KB1, cb = q % CB1, u = q / CB1;
        const int k0 = f % KB1, k1 = min(KB1, k0 + (fe - f));
        const int e = T.experts[u];
        float acc[2][2][NB8][4];
#pragma unroll
        for (int pa = 0; pa < 2; ++pa)
#pragma unroll
          for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int n = 0; n < NB8; ++n)
#pragma unroll
              for (int i = 0; i < 4; ++i) acc[pa][a][n][i] = 0.f;
        const int rt_up = ((64 * cb) & 127) + 16 * w, rt_gate = ((P.I + 64 * cb) & 127) + 16 * w;
        const unsigned octets = NB8 == 1 ? 1u : T.omask[u];
        for (int kb = k0; kb < k1; ++kb) {
          const int slot = 2 * si + grp;
          TIMER_START(t0);
          if (!mbar_wait(&T.full[slot], ph, &T.abort_flag)) *P.status = ST_TIMEOUT_FULL;
          TIMER_ADD(tm_wait, t0);
          TIMER_START(t1);
          const uint32_t st = ring_a + slot * kSlotBytes;
          mma_tile<NB8>(st, 16 * w, 64 + 16 * w, st + kCodesBytes, rt_up, st + kCodesBytes + 2048, rt_gate,
                        4 * kb + t < P.KT1, region_a + kb * (NB8 * 4096), lane, octets, acc);
          __syncwarp();
          if (lane == 0) mbar_arrive(&T.empty[slot]);
          if (++si == per) { si = 0; ph ^= 1u; }
          TIMER_ADD(tm_mma, t1);
        }
        TIMER_START(t2);
        float r[8 * NB8];   // [rb][n][4]: rb 0 = up, rb 1 = gate
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
          for (int n = 0; n < NB8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) r[(a * NB8 + n) * 4 + i] = acc[0][a][n][i] + acc[1][a][n][i];
        const int piece_first = f;
        f += k1 - k0;
        // ---- finish the unit: directly when this piece covers all of K, else through the scratch and a last arriver
        bool finalize = true;
        if (!(k0 == 0 && k1 == KB1)) {
          const int slot_id = piece_first == fs ? 0 : 1;
          float* mine = P.scratch + ((long long)(v * 2 + slot_id) * kGroupThreads + gtid) * 16;
#pragma unroll
          for (int i = 0; i < 2 * NB8; ++i)
            *reinterpret_cast<float4*>(mine + 4 * i) = make_float4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
          named_bar_sync(1 + grp, kGroupThreads);
          const int vlo = worker_of(q * KB1, T1, V), vhi = worker_of(q * KB1 + KB1 - 1, T1, V);
          if (gtid == 0) {
            __threadfence();   // cumulative: orders the group's stores (observed through the barrier) before the arrival
            int nlive = 0;
            for (int pv = vlo; pv <= vhi; ++pv) nlive += T.sb1[pv + 1] > T.sb1[pv];
            const unsigned old = atomicAdd(P.cnt1 + q, 1u);
            const int last = old + 1u == (unsigned)nlive;
            if (last) { P.cnt1[q] = 0; __threadfence(); }
            T.last_flag[grp] = last;
          }
          named_bar_sync(1 + grp, kGroupThreads);
          finalize = T.last_flag[grp] != 0;
          if (finalize) {
            reduce_pieces<NB8>(P.scratch, T.sb1, q * KB1, vlo, vhi, gtid, r);
          }
          named_bar_sync(1 + grp, kGroupThreads);   // last_flag may be rewritten by the next unit only after all read it
        }
        if (finalize) {
          const float alpha = P.alpha1[e];
          __half* af = P.actfrag + (long long)u * KB2 * (NB8 * 2048);
#pragma unroll
          for (int n = 0; n < NB8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int tok = 8 * n + 2 * t + (i & 1);
              const int c = 64 * cb + 16 * w + g + ((i >> 1) << 3);   // intermediate column (K index of FC2)
              // is token tok routed to expert e, and through which pair?
              int pair = -1;
              if (tok < P.M)
                for (int s = 0; s < P.top_k; ++s)
                  if (T.ids[tok * P.top_k + s] == e) pair = tok * P.top_k + s;
              float a = 0.f;
              if (pair >= 0) {
                a = silu_mul(alpha * r[(NB8 + n) * 4 + i], alpha * r[n * 4 + i]);
                a = fminf(fmaxf(a, -65504.f), 65504.f);
              }
              af[frag_index<NB8>(c, tok)] = __float2half_rn(a);
              if (P.act_bf16 && pair >= 0)
                for (int s = 0; s < P.top_k; ++s)
                  if (T.ids[tok * P.top_k + s] == e) P.act_bf16[(long long)(tok * P.top_k + s) * P.I + c] = __float2bfloat16_rn(a);
            }
          if (cb == CB1 - 1 && (P.I & 255)) {   // zero the K padding of this expert's activation slabs
            for (int i = gtid; i < (KB2 * 256 - P.I) * 8 * NB8; i += kGroupThreads)
              af[frag_index<NB8>(P.I + i / (8 * NB8), i % (8 * NB8))] = __float2half_rn(0.f);
          }
        }
        TIMER_ADD(tm_fix, t2);
      }
      if (do2) {
        // ---- publish FC1's results and arrive at the grid-wide barrier (the producers are the only waiters)
        fence_proxy_async();
        named_bar_sync(1 + grp, kGroupThreads);
        if (gtid == 0) {
          __threadfence();
          const unsigned old = atomicAdd(P.gridbar, 1u);
          if (old == (unsigned)(V - 1)) {
            P.gridbar[0] = 0;
            __threadfence();
            atomicAdd(P.gridbar + 1, 1u);
          }
        }
      }
    }
#ifdef B200_TIMERS
    const long long tm_phase1 = clock64() - tm_begin;
#endif

    if (do2) {
      // ---- FC2 pieces of this worker: tiles ordered (output block nb, expert u, K box kb)
      const int fs = T.sb2[v], fe = T.sb2[v + 1];
      const int per_nb = U * KB2;
      int f = fs;
      while (f < fe) {
        const int nb = f / per_nb;
        const int pe = min(fe, (nb + 1) * per_nb);   // end of this piece
        float r[8 * NB8];   // [rb][n][4] running output sums of this piece
#pragma unroll
        for (int i = 0; i < 8 * NB8; ++i) r[i] = 0.f;
        const int piece_start = f;
        int kb = f % KB2, u = (f / KB2) % U;
        while (f < pe) {
          const int k1 = min(KB2, kb + (pe - f));
          const int e = T.experts[u];
          float acc[2][2][NB8][4];
#pragma unroll
          for (int pa = 0; pa < 2; ++pa)
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
              for (int n = 0; n < NB8; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[pa][a][n][i] = 0.f;
          f += k1 - kb;
          const unsigned octets = NB8 == 1 ? 1u : T.omask[u];
          for (; kb < k1; ++kb) {
            const int slot = 2 * si + grp;
            TIMER_START(t0);
            if (!mbar_wait(&T.full[slot], ph, &T.abort_flag)) *P.status = ST_TIMEOUT_FULL;
            TIMER_ADD(tm_wait, t0);
            TIMER_START(t1);
            const uint32_t st = ring_a + slot * kSlotBytes;
            mma_tile<NB8>(st, 32 * w, 32 * w + 16, st + kCodesBytes, 32 * w, st + kCodesBytes, 32 * w + 16,
                          4 * kb + t < P.KT2, region_a + slot * slab_bytes, lane, octets, acc);
            __syncwarp();
            if (lane == 0) mbar_arrive(&T.empty[slot]);
            if (++si == per) { si = 0; ph ^= 1u; }
            TIMER_ADD(tm_mma, t1);
          }
          // routing weight x alpha2 for this lane's token columns, applied in fp32
          const float alpha = P.alpha2[e];
#pragma unroll
          for (int n = 0; n < NB8; ++n)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
              const int tok = 8 * n + 2 * t + c;
              float sc = 0.f;
              if (tok < P.M)
                for (int s = 0; s < P.top_k; ++s)
                  if (T.ids[tok * P.top_k + s] == e) sc += T.wts[tok * P.top_k + s];
              sc *= alpha;
#pragma unroll
              for (int a = 0; a < 2; ++a) {
                r[(a * NB8 + n) * 4 + c] += sc * (acc[0][a][n][c] + acc[1][a][n][c]);
                r[(a * NB8 + n) * 4 + 2 + c] += sc * (acc[0][a][n][2 + c] + acc[1][a][n][2 + c]);
              }
            }
          if (kb == KB2) { kb = 0; ++u; }   // u wraps only at a piece boundary, where it is recomputed
        }
        // ---- every output block is shared by several workers: partial sums to the scratch, last arriver reduces
        {
          TIMER_START(t2);
          const int slot_id = piece_start == fs ? 0 : 1;
          float* mine = P.scratch + ((long long)(v * 2 + slot_id) * kGroupThreads + gtid) * 16;
#pragma unroll
          for (int i = 0; i < 2 * NB8; ++i)
            *reinterpret_cast<float4*>(mine + 4 * i) = make_float4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]);
          named_bar_sync(1 + grp, kGroupThreads);
          const int vlo = worker_of(nb * per_nb, T2, V), vhi = worker_of((nb + 1) * per_nb - 1, T2, V);
          if (gtid == 0) {
            __threadfence();
            int nlive = 0;
            for (int pv = vlo; pv <= vhi; ++pv) nlive += T.sb2[pv + 1] > T.sb2[pv];
            const unsigned old = atomicAdd(P.cnt2 + nb, 1u);
            const int last = old + 1u == (unsigned)nlive;
            if (last) { P.cnt2[nb] = 0; __threadfence(); }
            T.last_flag[grp] = last;
          }
          named_bar_sync(1 + grp, kGroupThreads);
          const bool last = T.last_flag[grp] != 0;
          if (last) {
            reduce_pieces<NB8>(P.scratch, T.sb2, nb * per_nb, vlo, vhi, gtid, r);
#pragma unroll
            for (int a = 0; a < 2; ++a)
#pragma unroll
              for (int n = 0; n < NB8; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const int tok = 8 * n + 2 * t + (i & 1);
                  const int row = 128 * nb + 32 * w + 16 * a + g + ((i >> 1) << 3);
                  if (tok < P.M) P.out[(long long)tok * P.H + row] = __float2bfloat16_rn(r[(a * NB8 + n) * 4 + i]);
                }
          }
          named_bar_sync(1 + grp, kGroupThreads);
          TIMER_ADD(tm_fix, t2);
        }
      }
    }
#ifdef B200_TIMERS
    if (P.debug && gtid == 0) {
      P.debug[v * 8 + 0] = tm_wait; P.debug[v * 8 + 1] = tm_mma; P.debug[v * 8 + 2] = tm_fix; P.debug[v * 8 + 3] = tm_phase1;
      P.debug[v * 8 + 7] = clock64() - tm_begin;
    }
#endif
  }
  // Every TMA copy this CTA issued has been consumed by a full-barrier wait above. If a bounded wait ran out (abort flag
  // set, status word written), give copies still in flight time to land before the CTA retires.
  __syncthreads();
  if (T.abort_flag)
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
}

// bf16 activations [P, I] (row = pair index) -> the fragment-ordered f16 buffer the FC2 phase streams. Used only by the
// stand-alone FC2 entry point; the fused layer writes that buffer from FC1's epilogue.
template <int NB8>
__global__ void __launch_bounds__(256) k_act_to_frag(const __nv_bfloat16* __restrict__ act, const int* __restrict__ ids,
                                                     const int* __restrict__ experts, int Umax, int M, int top_k, int I, int KB2,
                                                     __half* __restrict__ actfrag) {
  const int u = blockIdx.x;
  if (u >= Umax) return;
  const int e = experts[u];
  if (e < 0) return;
  const int kpad = KB2 * 256;
  for (int i = threadIdx.x; i < kpad * 8 * NB8; i += blockDim.x) {
    const int tok = i / kpad, k = i % kpad;
    float a = 0.f;
    if (tok < M && k < I)
      for (int s = 0; s < top_k; ++s)
        if (ids[tok * top_k + s] == e) a = __bfloat162float(act[(long long)(tok * top_k + s) * I + k]);
    a = fminf(fmaxf(a, -65504.f), 65504.f);
    actfrag[(long long)u * KB2 * (NB8 * 2048) + frag_index<NB8>(k, tok)] = __float2half_rn(a);
  }
}

}  // namespace b200

using namespace b200;

int b200_decode_smem_bytes(int NS, int region_bytes) { return 1024 + NS * kSlotBytes + region_bytes + (int)sizeof(Tables); }

int b200_decode_launch(const DecodeParams& p, int grid, int smem_bytes, cudaStream_t st) {
  void* args[] = {(void*)&p};
  const void* fn = p.M <= 8 ? (const void*)k_moe_decode<1> : (const void*)k_moe_decode<2>;
  static thread_local int configured[2] = {0, 0};
  const int which = p.M <= 8 ? 0 : 1;
  if (configured[which] < smem_bytes) {
    B200_CUDA_TRY(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    configured[which] = smem_bytes;
  }
  // One CTA per SM (shared memory allows no second one), so on an otherwise idle device every CTA is resident and the
  // grid-wide barrier inside the kernel can complete; its waits are bounded either way. A cooperative launch makes
  // co-residency a launch-time guarantee at the price of a few microseconds between back-to-back launches.
  if (p.cooperative) {
    B200_CUDA_TRY(cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(kThreads), args, (size_t)smem_bytes, st));
  } else {
    B200_CUDA_TRY(cudaLaunchKernel(fn, dim3(grid), dim3(kThreads), args, (size_t)smem_bytes, st));
  }
  return B200MOE_OK;
}

int b200_act_to_frag_launch(const void* act, const int* ids, const int* experts, int Umax, int M, int top_k, int I, int KB2,
                            void* actfrag, cudaStream_t st) {
  if (M <= 8)
    k_act_to_frag<1><<<Umax, 256, 0, st>>>((const __nv_bfloat16*)act, ids, experts, Umax, M, top_k, I, KB2, (__half*)actfrag);
  else
    k_act_to_frag<2><<<Umax, 256, 0, st>>>((const __nv_bfloat16*)act, ids, experts, Umax, M, top_k, I, KB2, (__half*)actfrag);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}
