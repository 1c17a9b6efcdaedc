// Kernel parameter block of the fused decode layer (passed by value as a __grid_constant__).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace b200 {

struct DecodeParams {
  CUtensorMap tm1;   // FC1 codes viewed u8 [E*2I rows, H/2 bytes], box 128 B x 64 rows, 128B swizzle
  CUtensorMap tm2;   // FC2 codes viewed u8 [E*H rows, I/2 bytes], box 128 B x 128 rows, 128B swizzle
  const uint8_t* s1;  // FC1 block scales, 128x4 swizzle per expert
  const uint8_t* s2;  // FC2 block scales, 128x4 swizzle per expert
  const float* alpha1;
  const float* alpha2;
  const __nv_bfloat16* x;   // [M, H]
  const int* ids;           // [M, top_k]
  const float* wts;         // [M, top_k]
  __nv_bfloat16* out;       // [M, H]
  __nv_bfloat16* act_bf16;  // optional [M*top_k, I], row = pair index
  __half* actfrag;          // workspace: FC1 output in the fragment order FC2 streams
  float* scratch;           // workspace: split-unit partial sums, 2 slots x 128 threads x 16 floats per worker
  unsigned* cnt1;           // workspace: arrival counters per FC1 unit (self-resetting)
  unsigned* cnt2;           // workspace: arrival counters per FC2 output block (self-resetting)
  unsigned* gridbar;        // workspace: [0] arrivals, [1] generation
  int* status;              // workspace: 0, or the code of the first bounded wait that ran out
  long long* debug;         // workspace: per-worker cycle counters (written only by the timer build)
  int* experts_out;         // optional routing tables in the reference's padded form
  int* offsets_out;
  int* pairs_out;
  long long s1_expert_stride, s2_expert_stride;
  int M, E, H, I, top_k, Umax;
  int phases;               // bit 0: FC1, bit 1: FC2
  int cooperative;          // launch with cudaLaunchCooperativeKernel
  int NS;                   // ring stages (even)
  int region_bytes;         // shared-memory region for x fragments / activation slabs
  int KB1, KB2;             // 256-code K boxes of FC1 (over H) and FC2 (over I)
  int CB1, NB2;             // 64-column blocks of FC1, 128-row blocks of FC2
  int KT1, KT2;             // 4-column scale tiles along K
};

// Parameter block of the tcgen05 decode kernel (k_moe_decode_tc).
struct DecodeTcParams {
  const uint8_t* w1t;        // FC1 tile records [E][I/64][KB1][18432]: codes image + scale tiles (k_pack_tiles)
  const uint8_t* w2t;        // FC2 tile records [E][H/128][KB2][18432]
  const float* alpha1;
  const float* alpha2;
  const float* alpha2_ref;   // [0] = max over experts of alpha2, [1] = its reciprocal
  const uint8_t* xb;         // expanded x operand: [KB1][N][128 B] images then [KT1][512] scale tiles
  const float* xscale;       // 1 / g_t per column of the x operand [N]
  uint8_t* aslab;            // expanded activations (FC2 operand): [Umax][KB2] slabs of N*128 + 2048 bytes
  const int* ids;
  const float* wts;
  __nv_bfloat16* out;
  float* scratch;
  unsigned* cnt1;
  unsigned* cnt2;
  unsigned long long* gates; // workspace: arrival counters of the two FC1 gates; only ever incremented, V per launch and gate
  int* status;               // workspace: [0] code of the first bounded wait that ran out / bad expert id, [1] activation range
                             // exceeded, [2] routing inputs changed under the call
  int* experts_out;
  int* offsets_out;
  int* pairs_out;
  long long* debug;          // per-worker cycle counters (timer build only), 16 per worker
  float act_g1;              // global scale of the first activation term
  int M, E, H, I, top_k, Umax;
  int NS, region_bytes;
  int KB1, KB2, CB1, NB2, KT1, KT2;
};

}  // namespace b200

int b200_decode_tc_smem_bytes(int NS, int region_bytes);
int b200_expand_x_launch(const void* x, int M, int H, int N, int KB1, void* xb, float* colscale, bool chained, cudaStream_t st);
int b200_pack_tiles_launch(const void* q, const void* sf, void* out, int E, int rows_per_expert, int row_bytes, int blocks, int KB, int KT,
                           int fc1, int I, long long sf_stride, cudaStream_t st);
int b200_decode_tc_launch(const b200::DecodeTcParams& p, int grid, int smem_bytes, bool chained, cudaStream_t st);
int b200_decode_smem_bytes(int NS, int region_bytes);
int b200_decode_launch(const b200::DecodeParams& p, int grid, int smem_bytes, cudaStream_t st);
int b200_act_to_frag_launch(const void* act, const int* ids, const int* experts, int Umax, int M, int top_k, int I, int KB2,
                            void* actfrag, cudaStream_t st);
