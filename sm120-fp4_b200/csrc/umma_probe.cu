// Single-tile check of the tcgen05 block-scaled FP4 MMA building blocks (TMEM allocation, shared-memory descriptors,
// scale-factor copies, kind::mxf4nvf4 MMA, accumulator loads): D[128, N] = dequant(A)[128, K] * dequant(B)[N, K]^T.
// One CTA, operands staged by ordinary stores in the layout a 128B-swizzled TMA box produces. It is the unit test of
// tcgen05.cuh; the two ways the kernels move block scales into TMEM (tcgen05.cp, or registers + tcgen05.st) can be selected.
#include "common.cuh"
#include "tcgen05.cuh"

namespace b200 {

struct ProbeKnobs {
  uint32_t op_lbo, op_sbo, op_layout;   // operand descriptor (bytes, bytes, layout type)
  uint32_t sf_lbo, sf_sbo;              // scale-tile descriptor; sf_sbo == 0: no tcgen05.cp - the four warps move the scale
                                        // tiles shared memory -> registers -> TMEM (tcgen05.st), each into its own lane quadrant
  uint32_t idesc;                       // 0: computed by idesc_mxf4nvf4
  uint32_t k_step;                      // descriptor start-address increment per K=64 step, in 16-byte units
  uint32_t sf_col_step;                 // TMEM columns per K=64 step of scale factors
};

__global__ void __launch_bounds__(128, 1) k_umma_probe(const uint8_t* __restrict__ a, const uint8_t* __restrict__ sfa,
                                                       const uint8_t* __restrict__ b, const uint8_t* __restrict__ sfb, int N, int K,
                                                       float* __restrict__ d, ProbeKnobs kn, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int nkb = K / 256;
  uint8_t* sA = smem;                          // [nkb][128 rows][128 B], 128B swizzle
  uint8_t* sB = sA + nkb * 16384;              // [nkb][128 rows][128 B] (rows >= N zero)
  uint8_t* sSFA = sB + nkb * 16384;            // [nkb*4][512 B]
  uint8_t* sSFB = sSFA + nkb * 2048;
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  __shared__ volatile int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  if (tid == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base, 256);
    tmem_relinquish();
  }
  // stage the operands: element (row, byte c) of a 128-byte row goes to row*128 + ((c/16 ^ (row&7))*16) + c%16
  const int row_bytes = K / 2;
  for (int i = tid; i < nkb * 128 * 8; i += 128) {
    const int kb = i / 1024, r = (i / 8) % 128, ch = i % 8;
    const uint4 va = *reinterpret_cast<const uint4*>(a + (long long)r * row_bytes + kb * 128 + ch * 16);
    uint4 vb = make_uint4(0u, 0u, 0u, 0u);
    if (r < N) vb = *reinterpret_cast<const uint4*>(b + (long long)r * row_bytes + kb * 128 + ch * 16);
    const int off = kb * 16384 + r * 128 + ((ch ^ (r & 7)) << 4);
    *reinterpret_cast<uint4*>(sA + off) = va;
    *reinterpret_cast<uint4*>(sB + off) = vb;
  }
  for (int i = tid; i < nkb * 2048 / 16; i += 128) {
    reinterpret_cast<uint4*>(sSFA)[i] = reinterpret_cast<const uint4*>(sfa)[i];
    reinterpret_cast<uint4*>(sSFB)[i] = reinterpret_cast<const uint4*>(sfb)[i];
  }
  fence_proxy_async();          // generic-proxy stores -> visible to the tensor-core (async) proxy
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = tmem_base;
  const uint32_t d_tmem = tb, sfa_tmem = tb + 128, sfb_tmem = tb + 192;
  const bool sf_by_st = kn.sf_sbo == 0;
  if (sf_by_st) {               // lane l of every quadrant holds row l of each 512-byte tile: 16 bytes = 4 columns
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int kb = 0; kb < nkb; ++kb) {
      uint32_t ra[16], rb[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 va = lds128(smem_u32(sSFA + (kb * 4 + j) * 512 + (tid & 31) * 16));
        const uint4 vb = lds128(smem_u32(sSFB + (kb * 4 + j) * 512 + (tid & 31) * 16));
        ra[4 * j] = va.x, ra[4 * j + 1] = va.y, ra[4 * j + 2] = va.z, ra[4 * j + 3] = va.w;
        rb[4 * j] = vb.x, rb[4 * j + 1] = vb.y, rb[4 * j + 2] = vb.z, rb[4 * j + 3] = vb.w;
      }
      tmem_st_32x32b_x16(sfa_tmem + 16 * kb + lane_base, ra);
      tmem_st_32x32b_x16(sfb_tmem + 16 * kb + lane_base, rb);
    }
    tmem_st_wait();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  if (tid == 32) {              // one thread issues all tensor-core work
    const uint32_t idesc = kn.idesc ? kn.idesc : idesc_mxf4nvf4(128, N);
    for (int kb = 0; kb < nkb; ++kb)
      for (int j = 0; j < 4; ++j) {
        const int s = kb * 4 + j;
        if (!sf_by_st) {
          tmem_cp_sf(sfa_tmem + s * kn.sf_col_step, smem_desc(smem_u32(sSFA + s * 512), kn.sf_lbo, kn.sf_sbo, 0));
          tmem_cp_sf(sfb_tmem + s * kn.sf_col_step, smem_desc(smem_u32(sSFB + s * 512), kn.sf_lbo, kn.sf_sbo, 0));
        }
        const uint64_t ad = smem_desc(smem_u32(sA + kb * 16384), kn.op_lbo, kn.op_sbo, kn.op_layout) + (uint64_t)(j * kn.k_step);
        const uint64_t bd = smem_desc(smem_u32(sB + kb * 16384), kn.op_lbo, kn.op_sbo, kn.op_layout) + (uint64_t)(j * kn.k_step);
        umma_mxf4nvf4(d_tmem, ad, bd, idesc, sfa_tmem + s * kn.sf_col_step, sfb_tmem + s * kn.sf_col_step, s != 0);
      }
    umma_commit(&bar);
  }
  if (!mbar_wait(&bar, 0, &abort_flag, 1u << 18)) *status = 1;
  tc_fence_after();
  if (!abort_flag) {
    for (int c0 = 0; c0 < N; c0 += 16) {
      uint32_t r[16];
      tmem_ld_32x32b_x16(d_tmem + ((uint32_t)(warp * 32) << 16) + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) d[(long long)tid * N + c0 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 256);
}


// The same check for a CTA pair (cta_group::2): D[256, 128] = dequant(A)[256, K] * dequant(B)[128, K]^T. A cluster of two CTAs:
// CTA r stages A rows 128r.., the scale tiles of those rows, B rows 64r.. and the scale tiles of ALL 128 B rows (every CTA of
// the pair keeps the B scales of the whole N in its own TMEM); scales go through registers; the leader issues the MMAs and one
// commit that arrives on both CTAs' barriers; each CTA reads its own 128 accumulator rows.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1)
    k_umma2_probe(const uint8_t* __restrict__ a, const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ b, const uint8_t* __restrict__ sfb,
                  int K, float* __restrict__ d, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  const int nkb = K / 256;
  uint8_t* sA = smem;                          // [nkb][128 rows][128 B]
  uint8_t* sB = sA + nkb * 16384;              // [nkb][64 rows][128 B]
  uint8_t* sSFA = sB + nkb * 8192;             // [nkb*4][512 B]
  uint8_t* sSFB = sSFA + nkb * 2048;
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  __shared__ volatile int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  const uint32_t rank = cluster_ctarank();
  if (tid == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc2(&tmem_base, 256);
    tmem_relinquish2();
  }
  const int row_bytes = K / 2;
  for (int i = tid; i < nkb * 128 * 8; i += 128) {
    const int kb = i / 1024, r = (i / 8) % 128, ch = i % 8;
    const uint4 va = *reinterpret_cast<const uint4*>(a + (long long)(128 * rank + r) * row_bytes + kb * 128 + ch * 16);
    *reinterpret_cast<uint4*>(sA + kb * 16384 + r * 128 + ((ch ^ (r & 7)) << 4)) = va;
    if (r < 64) {
      const uint4 vb = *reinterpret_cast<const uint4*>(b + (long long)(64 * rank + r) * row_bytes + kb * 128 + ch * 16);
      *reinterpret_cast<uint4*>(sB + kb * 8192 + r * 128 + ((ch ^ (r & 7)) << 4)) = vb;
    }
  }
  for (int i = tid; i < nkb * 2048 / 16; i += 128) {
    reinterpret_cast<uint4*>(sSFA)[i] = reinterpret_cast<const uint4*>(sfa + (long long)rank * nkb * 2048)[i];   // row block `rank` of the 128x4 layout
    reinterpret_cast<uint4*>(sSFB)[i] = reinterpret_cast<const uint4*>(sfb)[i];
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = tmem_base;
  const uint32_t d_tmem = tb, sfa_tmem = tb + 128, sfb_tmem = tb + 192;
  {
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int kb = 0; kb < nkb; ++kb) {
      uint32_t ra[16], rb[16];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 va = lds128(smem_u32(sSFA + (kb * 4 + j) * 512 + (tid & 31) * 16));
        const uint4 vb = lds128(smem_u32(sSFB + (kb * 4 + j) * 512 + (tid & 31) * 16));
        ra[4 * j] = va.x, ra[4 * j + 1] = va.y, ra[4 * j + 2] = va.z, ra[4 * j + 3] = va.w;
        rb[4 * j] = vb.x, rb[4 * j + 1] = vb.y, rb[4 * j + 2] = vb.z, rb[4 * j + 3] = vb.w;
      }
      tmem_st_32x32b_x16(sfa_tmem + 16 * kb + lane_base, ra);
      tmem_st_32x32b_x16(sfb_tmem + 16 * kb + lane_base, rb);
    }
    tmem_st_wait();
  }
  tc_fence_before();
  cluster_sync_all();          // both CTAs' operands and scales are in place
  tc_fence_after();
  if (rank == 0 && warp == 1) {
    const uint32_t el = elect_one();
    const uint32_t idesc = idesc_mxf4nvf4_pair(128);
    for (int kb = 0; kb < nkb; ++kb)
      for (int j = 0; j < 4; ++j) {
        const uint64_t ad = smem_desc_sw128_kmajor(smem_u32(sA + kb * 16384)) + (uint64_t)(2 * j);
        const uint64_t bd = smem_desc_sw128_kmajor(smem_u32(sB + kb * 8192)) + (uint64_t)(2 * j);
        umma2_mxf4nvf4_p(d_tmem, ad, bd, idesc, sfa_tmem + 16 * kb + 4 * j, sfb_tmem + 16 * kb + 4 * j, (kb | j) != 0, el);
      }
    umma2_commit_p(&bar, (uint16_t)3, el);
  }
  if (!mbar_wait(&bar, 0, &abort_flag, 1u << 18)) status[rank] = 1;
  tc_fence_after();
  if (!abort_flag) {
    for (int c0 = 0; c0 < 128; c0 += 16) {
      uint32_t r[16];
      tmem_ld_32x32b_x16(d_tmem + ((uint32_t)(warp * 32) << 16) + c0, r);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 16; ++i) d[(long long)(128 * rank + tid) * 128 + c0 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  cluster_sync_all();          // nobody frees TMEM while the peer may still be read by the pair's MMAs
  if (warp == 0) tmem_dealloc2(tb, 256);
}

#ifdef B200_DIAGNOSTICS
// Issue-cost measurement of the tcgen05 operations the kernels use: `reps` rounds of {ncp scale copies, nmma MMAs of
// shape 128 x N x 64, ncommit commits}, timed with clock64 around issue and around issue + completion.
// flags: 1 = alternate between two accumulators; 2 = every round also waits on an mbarrier whose phase completed long
// ago; 4 = every round executes tcgen05.fence::after_thread_sync; 8 = every round waits for its own commit (commit ->
// arrive latency; needs ncommit >= 1); 16 = the copies are issued by a second thread in another warp, concurrently with
// the MMAs of the first (cycles[2], cycles[3] are the second thread's issue and completion times); 32 = the issuing
// warps stay converged and one elected lane issues (predicated instructions) instead of a single diverged thread.
__global__ void __launch_bounds__(128, 1) k_umma_cost(int N, int reps, int ncp, int nmma, int flags, int ncommit, long long* __restrict__ cycles) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar, bar2, bar_done, bar_b, bar_b2;
  __shared__ uint32_t tmem_base;
  __shared__ volatile int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < (32768 + 4096) / 16; i += 128) reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
  if (tid == 0) {
    mbar_init(&bar, 1); mbar_init(&bar2, 1); mbar_init(&bar_done, 1); mbar_init(&bar_b, 1); mbar_init(&bar_b2, 1);
    abort_flag = 0;
    fence_mbar_init();
    mbar_arrive(&bar_done);   // phase 0 of this barrier is complete from here on
  }
  if (warp == 0) { tmem_alloc(&tmem_base, 512); tmem_relinquish(); }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = tmem_base;
  const bool split = (flags & 16) != 0;
  if ((flags & 32) && (warp == 1 || (split && warp == 2))) {
    const bool second = warp == 2;
    const uint32_t el = elect_one();
    const uint32_t idesc = idesc_mxf4nvf4(128, N);
    const uint32_t sA = smem_u32(smem), sB = smem_u32(smem + 16384), sS = smem_u32(smem + 32768);
    uint64_t* round_bar = second ? &bar_b2 : &bar2;
    uint64_t* end_bar = second ? &bar_b : &bar;
    const int my_cp = split ? (second ? ncp : 0) : ncp, my_mma = second ? 0 : nmma;
    uint32_t ph = 0;
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
      if (flags & 2) mbar_wait(&bar_done, 0, &abort_flag, 1u << 16);
      if (flags & 4) tc_fence_after();
      for (int c = 0; c < my_cp; ++c) tmem_cp_sf_p(tb + 256 + 4 * (c & 31), smem_desc_sf_tile(sS + (c & 7) * 512), el);
      for (int m = 0; m < my_mma; ++m)
        umma_mxf4nvf4_p(tb + ((flags & 1) ? 128 * (m & 1) : 0), smem_desc_sw128_kmajor(sA) + 2 * (m & 3), smem_desc_sw128_kmajor(sB) + 2 * (m & 3), idesc,
                        tb + 256 + 4 * (m & 3), tb + 272 + 4 * (m & 3), 1u, el);
      for (int c = 0; c < ncommit; ++c) umma_commit_p(round_bar, el);
      if ((flags & 8) && ncommit == 1) { mbar_wait(round_bar, ph, &abort_flag, 1u << 20); ph ^= 1u; }
    }
    const long long t1 = clock64();
    umma_commit_p(end_bar, el);
    mbar_wait(end_bar, 0, &abort_flag, 1u << 22);
    const long long t2 = clock64();
    if ((tid & 31) == 0) {
      cycles[second ? 2 : 0] = t1 - t0;
      cycles[second ? 3 : 1] = t2 - t0;
    }
  } else if (!(flags & 32) && (tid == 32 || (split && tid == 64))) {
    const bool second = tid == 64;
    const uint32_t idesc = idesc_mxf4nvf4(128, N);
    const uint32_t sA = smem_u32(smem), sB = smem_u32(smem + 16384), sS = smem_u32(smem + 32768);
    uint64_t* round_bar = second ? &bar_b2 : &bar2;
    uint64_t* end_bar = second ? &bar_b : &bar;
    const int my_cp = split ? (second ? ncp : 0) : ncp, my_mma = second ? 0 : nmma;
    uint32_t ph = 0;
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
      if (flags & 2) mbar_wait(&bar_done, 0, &abort_flag, 1u << 16);
      if (flags & 4) tc_fence_after();
      for (int c = 0; c < my_cp; ++c) tmem_cp_sf(tb + 256 + 4 * (c & 31), smem_desc_sf_tile(sS + (c & 7) * 512));
      for (int m = 0; m < my_mma; ++m)
        umma_mxf4nvf4(tb + ((flags & 1) ? 128 * (m & 1) : 0), smem_desc_sw128_kmajor(sA) + 2 * (m & 3), smem_desc_sw128_kmajor(sB) + 2 * (m & 3), idesc,
                      tb + 256 + 4 * (m & 3), tb + 272 + 4 * (m & 3), 1u);
      for (int c = 0; c < ncommit; ++c) umma_commit(round_bar);
      if ((flags & 8) && ncommit == 1) { mbar_wait(round_bar, ph, &abort_flag, 1u << 20); ph ^= 1u; }
    }
    const long long t1 = clock64();
    umma_commit(end_bar);
    mbar_wait(end_bar, 0, &abort_flag, 1u << 22);
    const long long t2 = clock64();
    cycles[second ? 2 : 0] = t1 - t0;
    cycles[second ? 3 : 1] = t2 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tb, 512);
}

#endif  // B200_DIAGNOSTICS

}  // namespace b200

using namespace b200;

#ifdef B200_DIAGNOSTICS
// cycles_dev: device int64 x 4 = {issue, completion} cycles of the first and (flags & 16) of the second issuing thread
extern "C" int b200moe_umma_cost(int N, int reps, int ncp, int nmma, int flags, int ncommit, long long* cycles_dev, void* stream) {
  if (!cycles_dev || N < 16 || N > 128 || N % 16 || reps < 1 || reps > 4096 || ncp < 0 || ncp > 64 || nmma < 0 || nmma > 64 || ncommit < 0 || ncommit > 8 || flags < 0 || flags > 63) return B200MOE_ERR_ARG;
  const int smem = 1024 + 32768 + 4096;
  B200_CUDA_TRY(cudaFuncSetAttribute(k_umma_cost, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  k_umma_cost<<<1, 128, smem, (cudaStream_t)stream>>>(N, reps, ncp, nmma, flags, ncommit, cycles_dev);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}
#endif  // B200_DIAGNOSTICS

// a u8 [128, K/2], sfa u8 128x4-swizzled over [128, K/16], b u8 [N, K/2], sfb u8 128x4-swizzled over [N -> 128, K/16],
// d f32 [128, N]; N a multiple of 16 up to 128, K a multiple of 256 up to 1024. scale_path: 0 = block scales copied into
// TMEM by tcgen05.cp, 1 = through registers by tcgen05.st (the path the layer kernels use). Nothing else is accepted: the
// descriptor fields themselves are fixed to the two encodings the library uses.
extern "C" int b200moe_umma_probe(const void* a, const void* sfa, const void* b, const void* sfb, int N, int K, float* d,
                                  int scale_path, int* status_dev, void* stream) {
  if (!a || !sfa || !b || !sfb || !d || !status_dev) return B200MOE_ERR_ARG;
  if (N < 16 || N > 128 || N % 16 || K < 256 || K > 1024 || K % 256) return B200MOE_ERR_SHAPE;
  if (scale_path != 0 && scale_path != 1) return B200MOE_ERR_ARG;
  const ProbeKnobs kn = scale_path == 0 ? ProbeKnobs{16, 1024, 2, 0, 128, 0, 2, 4} : ProbeKnobs{16, 1024, 2, 0, 0, 0, 2, 4};
  const int nkb = K / 256;
  const int smem = 1024 + nkb * (16384 * 2 + 4096);
  B200_CUDA_TRY(cudaFuncSetAttribute(k_umma_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  k_umma_probe<<<1, 128, smem, (cudaStream_t)stream>>>((const uint8_t*)a, (const uint8_t*)sfa, (const uint8_t*)b, (const uint8_t*)sfb, N, K,
                                                        d, kn, status_dev);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// The CTA-pair form: a u8 [256, K/2], sfa u8 128x4-swizzled over [256, K/16], b u8 [128, K/2], sfb u8 128x4-swizzled over
// [128, K/16], d f32 [256, 128], status int32 [2] (one word per CTA of the pair); K a multiple of 256 up to 1024.
extern "C" int b200moe_umma_pair_probe(const void* a, const void* sfa, const void* b, const void* sfb, int K, float* d, int* status_dev,
                                       void* stream) {
  if (!a || !sfa || !b || !sfb || !d || !status_dev) return B200MOE_ERR_ARG;
  if (K < 256 || K > 1024 || K % 256) return B200MOE_ERR_SHAPE;
  const int nkb = K / 256;
  const int smem = 1024 + nkb * (16384 + 8192 + 4096);
  B200_CUDA_TRY(cudaFuncSetAttribute(k_umma2_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  k_umma2_probe<<<2, 128, smem, (cudaStream_t)stream>>>((const uint8_t*)a, (const uint8_t*)sfa, (const uint8_t*)b, (const uint8_t*)sfb, K, d,
                                                         status_dev);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}
