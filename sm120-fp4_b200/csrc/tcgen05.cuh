// tcgen05 (5th-generation tensor core) wrappers for sm_100a: TMEM allocation, shared-memory matrix descriptors, the
// block-scaled FP4 MMA (kind::mxf4nvf4, E2M1 x E2M1 with UE4M3 scales per 16 elements), scale-factor copies into TMEM,
// accumulator loads. Descriptor bit layouts follow the public PTX ISA tables for tcgen05 matrix/instruction descriptors.
#pragma once
#include "ptx.cuh"

namespace b200 {

// ---------------------------------------------------------------------------------------------------- TMEM
// Whole-warp (.sync.aligned) allocation of `ncols` (power of two >= 32) TMEM columns; the base address lands in smem.
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor: start address, leading / stride byte offsets (all >> 4), version 1 (sm_100),
// layout type in bits 61..63 (0 = no swizzle, 2 = 128-byte swizzle).
__host__ __device__ __forceinline__ uint64_t smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type) {
  return (uint64_t)((smem_addr >> 4) & 0x3FFF) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | ((uint64_t)(layout_type & 7) << 61);
}
// K-major operand tile written by TMA with CU_TENSOR_MAP_SWIZZLE_128B: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128_kmajor(uint32_t smem_addr) { return smem_desc(smem_addr, 16, 1024, 2); }
// One 128x4 scale tile (512 bytes: 32 rows x 16 bytes, no swizzle): 8-row core matrices 128 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sf_tile(uint32_t smem_addr) { return smem_desc(smem_addr, 0, 128, 0); }

// Instruction descriptor of kind::mxf4nvf4 block-scaled MMA: A, B = E2M1 (format code 1), both K-major, UE4M3 scales,
// N >> 3 at bit 17, M >> 4 at bit 24; scale-factor ids zero (scale_vec::4X uses all four bytes of a TMEM word).
__host__ __device__ __forceinline__ uint32_t idesc_mxf4nvf4(int M, int N) {
  return (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | (0u << 23) | ((uint32_t)(M >> 4) << 24);
}

// ---------------------------------------------------------------------------------------------------- issue (one thread)
// D[tmem] (+)= A[smem] * B[smem], 128 x N x 64 FP4 with per-16 UE4M3 scales read from TMEM.
__device__ __forceinline__ void umma_mxf4nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                              uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// 512-byte scale tile (32 rows x 128 bits) from shared memory into 4 TMEM columns, replicated to all four lane quadrants.
__device__ __forceinline__ void tmem_cp_sf(uint32_t taddr, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
// mbarrier arrives once every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---------------------------------------------------------------------------------------------------- issue (whole warp)
// The same operations for a warp that stays converged: every lane executes the surrounding code with warp-uniform
// values, and `pred` (from elect_one) lets exactly one lane issue. Uniform operands can then live in uniform registers,
// which makes the issue much cheaper than from a single diverged lane.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred;
}
__device__ __forceinline__ void umma_mxf4nvf4_p(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                                uint32_t sfb_tmem, uint32_t accumulate, uint32_t pred) {
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.b32 p, %4, 0;\n setp.ne.b32 q, %7, 0;\n"
      " @q tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(pred)
      : "memory");
}
__device__ __forceinline__ void tmem_cp_sf_p(uint32_t taddr, uint64_t sdesc, uint32_t pred) {
  asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n @q tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;\n}\n" ::"r"(taddr), "l"(sdesc), "r"(pred) : "memory");
}
__device__ __forceinline__ void umma_commit_p(uint64_t* bar, uint32_t pred) {
  asm volatile("{\n .reg .pred q;\n setp.ne.b32 q, %1, 0;\n @q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n}\n" ::"r"(smem_u32(bar)), "r"(pred) : "memory");
}

// ---------------------------------------------------------------------------------------------------- accumulator loads
// 32 lanes (this warp's quadrant) x 32 consecutive fp32 columns -> 32 registers per thread (thread = lane = row).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// 16 registers per thread -> 16 consecutive columns of this warp's lane quadrant (thread = lane).
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 2i and 2i + 1) act as one tensor-core unit: an MMA of 256 x N x 64 whose A rows and
// accumulator rows are split 128 / 128 over the two CTAs' shared memory and TMEM, and whose B rows (N) are split N/2 / N/2
// over the two CTAs' shared memory, at the same CTA-relative offsets. The even CTA (the leader) issues; both allocate and free.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_sync_all() { cluster_arrive(); cluster_wait(); }
// the address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
// Arrival on a barrier of another CTA of the cluster. Default semantics (release at CTA scope): what the waiter consumes
// after these arrivals is tensor memory written by tcgen05.st / read by tcgen05.ld, ordered by tcgen05.wait and the
// tcgen05 fences on either side, never ordinary memory of the arriving CTA - and a release at cluster scope costs the
// arriving warp about a microsecond per arrival.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(remote_bar_addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {   // acquire at cluster scope
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t limit = (1u << 20)) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((it & 63u) == 63u) {
      if (*abort_flag) return false;
      if (it > 4096u) __nanosleep(64);
    }
  }
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ uint32_t idesc_mxf4nvf4_pair(int N) { return idesc_mxf4nvf4(256, N); }
// D[tmem of both CTAs] (+)= A[256 rows over both CTAs] * B[N rows over both CTAs]; issued by the leader CTA only
__device__ __forceinline__ void umma2_mxf4nvf4_p(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t sfa_tmem,
                                                 uint32_t sfb_tmem, uint32_t accumulate, uint32_t pred) {
  asm volatile(
      "{\n .reg .pred p, q;\n setp.ne.b32 p, %4, 0;\n setp.ne.b32 q, %7, 0;\n"
      " @q tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem), "r"(pred)
      : "memory");
}
// the mbarrier at this CTA-relative address arrives in every CTA of `cta_mask` (bit = cluster rank) once the pair's
// tensor-core operations issued so far have completed (a commit with multicast; no data is multicast)
__device__ __forceinline__ void umma2_commit_p(uint64_t* bar, uint16_t cta_mask, uint32_t pred) {
  asm volatile(
      "{\n .reg .pred q;\n setp.ne.b32 q, %2, 0;\n"
      " @q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n}\n"
      ::"r"(smem_u32(bar)), "h"(cta_mask), "r"(pred)
      : "memory");
}

}  // namespace b200
