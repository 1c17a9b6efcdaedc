// C ABI of the library: layer handle (tensor maps + geometry), workspace layout, decode entry points.
// No torch types, no exceptions, no device allocation: every device buffer is the caller's.
#include "common.cuh"
#include "decode_params.h"
#include <cudaTypedefs.h>
#include <stdlib.h>
#include <string.h>
#include <new>

namespace b200 {
thread_local cudaError_t g_last_cuda_error = cudaSuccess;

static PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = (PFN_cuTensorMapEncodeTiled_v12000)p;
  }
  return fn;
}

// u8 matrix [rows, row_bytes] -> tensor map with a 128-byte x box_rows box, 128B shared-memory swizzle, zero OOB fill.
__global__ void k_alpha_ref(const float* __restrict__ alpha, int E, float* __restrict__ out) {
  float m = 0.f;
  for (int e = 0; e < E; ++e) m = fmaxf(m, fabsf(alpha[e]));
  m = fmaxf(m, 1e-30f);
  out[0] = m;
  out[1] = 1.0f / m;
}

static int make_codes_map(CUtensorMap* map, const void* base, long long rows, long long row_bytes, int box_rows) {
  auto enc = tensor_map_encoder();
  if (!enc) return B200MOE_ERR_DEVICE;
  if (((uintptr_t)base & 15) || (row_bytes & 15)) return B200MOE_ERR_ARG;
  cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
  cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200MOE_OK : B200MOE_ERR_CUDA;
}
}  // namespace b200

using namespace b200;

struct b200moe_layer {
  int E, H, I, top_k;
  int sms;
  const void *q1, *s1, *q2, *s2;
  const float *alpha1, *alpha2;
  CUtensorMap tm1, tm2;
  int KB1, KB2, CB1, NB2, KT1, KT2;
  long long s1_stride, s2_stride;
  // workspace layout (byte offsets)
  long long off_status, off_cnt1, off_cnt2, off_scratch, off_actfrag, off_tables, off_actbf16, off_debug, off_hstage, ws_bytes;
  long long off_xb, off_xscale, off_aslab;   // operands of the tcgen05 decode kernel
  int umax_cap;
  // tcgen05 decode path: composed FC1 scale tiles + alpha2 reference in a caller-owned buffer (b200moe_layer_prepack)
  const uint8_t* w1t;
  const uint8_t* w2t;
  const float* alpha2_ref;
  long long prepack_bytes;
  int device;           // CUDA device the layer was created on
  int decode_impl;      // 0 auto (tcgen05 when prepacked), 1 legacy mma.sync kernel, 2 tcgen05 kernel
  float act_g1;
};

static inline long long align_up(long long v, long long a) { return (v + a - 1) / a * a; }

extern "C" int b200moe_version(void) { return 100; }

extern "C" const char* b200moe_error_string(int code) {
  switch (code) {
    case B200MOE_OK: return "ok";
    case B200MOE_ERR_ARG: return "bad argument (null pointer, negative size or misaligned buffer)";
    case B200MOE_ERR_SHAPE: return "shape not taken by the kernels";
    case B200MOE_ERR_CUDA: return "CUDA call failed";
    case B200MOE_ERR_DEVICE: return "no sm_100 device or tensor-map driver entry point missing";
    case B200MOE_ERR_TIMEOUT: return "a bounded device-side wait ran out";
    case B200MOE_ERR_WORKSPACE: return "workspace too small";
    case B200MOE_ERR_LIMIT: return "size beyond the stated maximum";
    case B200MOE_ERR_RANGE: return "an intermediate activation exceeded the range of the activation scale (raise it with b200moe_layer_set_act_scale)";
    case B200MOE_ERR_ORDER: return "topk_ids / topk_weights changed while the call was running: they were still being written when it started";
    default: return "unknown error";
  }
}

extern "C" const char* b200moe_last_cuda_error(void) { return cudaGetErrorString(g_last_cuda_error); }

// Decode-layer handle. q1 u8 [E, 2I, H/2] rows [up ; gate]; s1 u8 [E, pad128(2I), pad4(H/16)] in the 128x4 swizzle;
// q2 u8 [E, H, I/2]; s2 u8 [E, pad128(H), pad4(I/16)] in the 128x4 swizzle; alpha f32 [E] (= 1 / global scale).
extern "C" int b200moe_layer_create(b200moe_layer** out, int E, int H, int I, int top_k, const void* q1, const void* s1_128x4,
                                    const float* alpha1, const void* q2, const void* s2_128x4, const float* alpha2) {
  if (!out || !q1 || !s1_128x4 || !alpha1 || !q2 || !s2_128x4 || !alpha2) return B200MOE_ERR_ARG;
  if (E <= 0 || E > 256 || top_k <= 0 || top_k > 16 || H <= 0 || I <= 0) return B200MOE_ERR_SHAPE;
  if (H % 128 || I % 64) return B200MOE_ERR_SHAPE;   // FC2 output blocks of 128 rows, FC1 column blocks of 64
  if (((uintptr_t)s1_128x4 & 15) || ((uintptr_t)s2_128x4 & 15)) return B200MOE_ERR_ARG;
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  cudaDeviceProp prop;
  B200_CUDA_TRY(cudaGetDeviceProperties(&prop, dev));
  if (prop.major != 10) return B200MOE_ERR_DEVICE;
  b200moe_layer* L = new (std::nothrow) b200moe_layer;
  if (!L) return B200MOE_ERR_ARG;
  memset(L, 0, sizeof(*L));
  L->E = E, L->H = H, L->I = I, L->top_k = top_k, L->sms = prop.multiProcessorCount, L->device = dev;
  L->q1 = q1, L->s1 = s1_128x4, L->q2 = q2, L->s2 = s2_128x4, L->alpha1 = alpha1, L->alpha2 = alpha2;
  L->KB1 = (H + 255) / 256, L->KB2 = (I + 255) / 256;
  L->CB1 = I / 64, L->NB2 = H / 128;
  L->KT1 = (H / 16 + 3) / 4, L->KT2 = (I / 16 + 3) / 4;
  L->s1_stride = align_up(2LL * I, 128) * L->KT1 * 4;
  L->s2_stride = align_up((long long)H, 128) * L->KT2 * 4;
  int rc = make_codes_map(&L->tm1, q1, (long long)E * 2 * I, H / 2, 64);
  if (rc == B200MOE_OK) rc = make_codes_map(&L->tm2, q2, (long long)E * H, I / 2, 128);
  if (rc != B200MOE_OK) { delete L; return rc; }
  // workspace
  const int V = 2 * L->sms;
  L->umax_cap = E < 16 * top_k ? E : 16 * top_k;
  long long o = 0;
  L->off_status = o, o += 256;                                               // status + grid barrier words
  L->off_cnt1 = o, o = align_up(o + (long long)L->umax_cap * L->CB1 * 4, 256);
  L->off_cnt2 = o, o = align_up(o + (long long)L->NB2 * 4, 256);
  L->off_scratch = o, o = align_up(o + (long long)V * 2 * 128 * 16 * 4, 256);
  L->off_actfrag = o, o = align_up(o + (long long)L->umax_cap * L->KB2 * 8192, 256);
  L->off_tables = o, o = align_up(o + (long long)(2 * L->umax_cap + 1 + 16 * top_k) * 4, 256);
  L->off_actbf16 = o, o = align_up(o + (long long)16 * top_k * I * 2, 256);
  L->off_debug = o, o = align_up(o + (long long)V * 16 * 8, 256);
  L->off_xb = o, o = align_up(o + (long long)L->KB1 * 64 * 128 + (long long)L->KT1 * 512, 256);
  L->off_xscale = o, o += 256;
  L->off_aslab = o, o = align_up(o + (long long)L->umax_cap * L->KB2 * (64 * 128 + 2048), 256);
  L->off_hstage = o, o = align_up(o + 2LL * 16 * H * 2 + 2LL * 16 * top_k * 4, 256);   // device copies of host-side inputs / output
  L->ws_bytes = o;
  L->prepack_bytes = (long long)E * ((long long)L->CB1 * L->KB1 + (long long)L->NB2 * L->KB2) * 18432 + 256;
  L->act_g1 = 8.0f;
  *out = L;
  return B200MOE_OK;
}

extern "C" void b200moe_layer_destroy(b200moe_layer* L) { delete L; }

extern "C" long long b200moe_layer_workspace_bytes(const b200moe_layer* L) { return L ? L->ws_bytes : B200MOE_ERR_ARG; }

// Zero the workspace (counters, barrier words, status, activation padding). Once after allocation, and again after a
// call that returned a timeout status.
extern "C" int b200moe_layer_workspace_init(const b200moe_layer* L, void* ws, long long ws_bytes, void* stream) {
  if (!L || !ws) return B200MOE_ERR_ARG;
  if (ws_bytes < L->ws_bytes) return B200MOE_ERR_WORKSPACE;
  B200_CUDA_TRY(cudaMemsetAsync(ws, 0, (size_t)L->ws_bytes, (cudaStream_t)stream));
  return B200MOE_OK;
}

// ---- tcgen05 decode path -------------------------------------------------------------------------------------------
extern "C" long long b200moe_layer_prepack_bytes(const b200moe_layer* L) { return L ? L->prepack_bytes : B200MOE_ERR_ARG; }

// Build the kernel-native copy the tcgen05 decode kernel streams - every weight tile as one contiguous 18 KB record (codes
// in their shared-memory image + scale tiles) - and the alpha2 normaliser into `buffer` (caller-owned device memory of b200moe_layer_prepack_bytes bytes that must
// outlive the handle). Once per layer, like the layout rotation the reference does at load (vllm_backend.py:193-206).
extern "C" int b200moe_layer_prepack(b200moe_layer* L, void* buffer, long long buffer_bytes, void* stream) {
  if (!L || !buffer) return B200MOE_ERR_ARG;
  if (buffer_bytes < L->prepack_bytes) return B200MOE_ERR_WORKSPACE;
  if ((uintptr_t)buffer & 255) return B200MOE_ERR_ARG;
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* w1t = (uint8_t*)buffer;
  uint8_t* w2t = w1t + (long long)L->E * L->CB1 * L->KB1 * 18432;
  int rc = b200_pack_tiles_launch(L->q1, L->s1, w1t, L->E, 2 * L->I, L->H / 2, L->CB1, L->KB1, L->KT1, 1, L->I, L->s1_stride, st);
  if (rc != B200MOE_OK) return rc;
  rc = b200_pack_tiles_launch(L->q2, L->s2, w2t, L->E, L->H, L->I / 2, L->NB2, L->KB2, L->KT2, 0, L->I, L->s2_stride, st);
  if (rc != B200MOE_OK) return rc;
  float* ref = (float*)(w2t + (long long)L->E * L->NB2 * L->KB2 * 18432);
  k_alpha_ref<<<1, 1, 0, st>>>(L->alpha2, L->E, ref);
  B200_LAUNCH_CHECK();
  L->w1t = w1t;
  L->w2t = w2t;
  L->alpha2_ref = ref;
  return B200MOE_OK;
}

// After prepack the tcgen05 paths (decode, mid-sized batches, W4A4 prefill) read only the tile records. A caller that does
// not need the mma.sync kernel or the stand-alone FC1 / FC2 entry points may then free the checkpoint-layout codes and
// scales (about half of the layer's memory); this makes the handle forget them, so that a later call that would need
// them fails with B200MOE_ERR_ARG instead of reading freed memory.
extern "C" int b200moe_layer_release_checkpoint(b200moe_layer* L) {
  if (!L) return B200MOE_ERR_ARG;
  if (!L->w1t) return B200MOE_ERR_ARG;   // nothing else to run from
  L->q1 = L->s1 = L->q2 = L->s2 = nullptr;
  if (L->decode_impl == 1) L->decode_impl = 0;
  return B200MOE_OK;
}

// 0: tcgen05 kernel when the layer is prepacked, else the mma.sync kernel; 1: mma.sync kernel; 2: tcgen05 kernel.
extern "C" int b200moe_layer_set_decode_impl(b200moe_layer* L, int impl) {
  if (!L || impl < 0 || impl > 2) return B200MOE_ERR_ARG;
  if (impl == 2 && !L->w1t) return B200MOE_ERR_ARG;
  if (impl == 1 && !L->q1) return B200MOE_ERR_ARG;   // checkpoint-layout weights were released
  L->decode_impl = impl;
  return B200MOE_OK;
}

// Global scale of the first NVFP4 term of the FC1->FC2 activations (default 8; 1 / the checkpoint's w2 input scale is the
// calibrated choice). Block maxima up to 2688 / scale are represented without saturation.
extern "C" int b200moe_layer_set_act_scale(b200moe_layer* L, float g1) {
  if (!L || !(g1 > 0.f)) return B200MOE_ERR_ARG;
  L->act_g1 = g1;
  return B200MOE_OK;
}

static int decode_tc(b200moe_layer* L, const void* x, const int* ids, const float* wts, int M, void* out, void* ws, bool chained, void* stream) {
  uint8_t* w = (uint8_t*)ws;
  cudaStream_t st = (cudaStream_t)stream;
  const int nbv = M <= 4 ? 0 : M <= 8 ? 1 : 2;
  const int N = 16 << nbv;
  int rc = b200_expand_x_launch(x, M, L->H, N, L->KB1, w + L->off_xb, (float*)(w + L->off_xscale), chained, st);
  if (rc != B200MOE_OK) return rc;
  DecodeTcParams p;
  memset(&p, 0, sizeof(p));
  p.w1t = L->w1t, p.w2t = L->w2t, p.alpha1 = L->alpha1, p.alpha2 = L->alpha2, p.alpha2_ref = L->alpha2_ref;
  p.xb = w + L->off_xb, p.xscale = (const float*)(w + L->off_xscale);
  p.aslab = w + L->off_aslab;
  p.ids = ids, p.wts = wts, p.out = (__nv_bfloat16*)out;
  p.scratch = (float*)(w + L->off_scratch);
  p.cnt1 = (unsigned*)(w + L->off_cnt1), p.cnt2 = (unsigned*)(w + L->off_cnt2);
  p.status = (int*)(w + L->off_status);
  p.gates = (unsigned long long*)(w + L->off_status + 128);
  p.experts_out = (int*)(w + L->off_tables);
  p.offsets_out = p.experts_out + L->umax_cap;
  p.pairs_out = p.offsets_out + L->umax_cap + 1;
  p.debug = (long long*)(w + L->off_debug);
  p.act_g1 = L->act_g1;
  p.M = M, p.E = L->E, p.H = L->H, p.I = L->I, p.top_k = L->top_k;
  p.Umax = L->E < M * L->top_k ? L->E : M * L->top_k;
  p.KB1 = L->KB1, p.KB2 = L->KB2, p.CB1 = L->CB1, p.NB2 = L->NB2, p.KT1 = L->KT1, p.KT2 = L->KT2;
  const int xb = L->KB1 * N * 128 + L->KT1 * 512, slab = N * 128 + 2048;
  int NS = 12;
  for (; NS >= 2; --NS) {
    const int region = (int)align_up(xb > NS * slab ? xb : NS * slab, 1024);
    if (b200_decode_tc_smem_bytes(NS, region) <= 227 * 1024 - 6144) { p.region_bytes = region; break; }   // room for static shared memory
  }
  if (NS < 2) return B200MOE_ERR_SHAPE;
  p.NS = NS;
  return b200_decode_tc_launch(p, L->sms, b200_decode_tc_smem_bytes(NS, p.region_bytes), chained, st);
}

static int decode_common(const b200moe_layer* L, const void* x, const int* ids, const float* wts, int M, void* out, void* act_bf16,
                         int phases, int write_tables, void* ws, long long ws_bytes, void* stream) {
  if (!L || !ids || !wts || !ws) return B200MOE_ERR_ARG;
  if (!L->q1) return B200MOE_ERR_ARG;   // the mma.sync kernel reads the checkpoint layout, which the caller released
  if ((phases & 1) && !x) return B200MOE_ERR_ARG;
  if ((phases & 2) && !out) return B200MOE_ERR_ARG;
  if (M < 0) return B200MOE_ERR_ARG;
  if (M > 16) return B200MOE_ERR_LIMIT;
  if (ws_bytes < L->ws_bytes) return B200MOE_ERR_WORKSPACE;
  if (((uintptr_t)ws & 255) || ((uintptr_t)x & 15)) return B200MOE_ERR_ARG;
  if (M == 0) return B200MOE_OK;
  if (2 * L->sms > 512) return B200MOE_ERR_DEVICE;   // share tables of the kernel hold 512 workers
  uint8_t* w = (uint8_t*)ws;
  DecodeParams p;
  memset(&p, 0, sizeof(p));
  p.tm1 = L->tm1, p.tm2 = L->tm2;
  p.s1 = (const uint8_t*)L->s1, p.s2 = (const uint8_t*)L->s2;
  p.alpha1 = L->alpha1, p.alpha2 = L->alpha2;
  p.x = (const __nv_bfloat16*)x, p.ids = ids, p.wts = wts, p.out = (__nv_bfloat16*)out;
  p.act_bf16 = (__nv_bfloat16*)act_bf16;
  p.actfrag = (__half*)(w + L->off_actfrag);
  p.scratch = (float*)(w + L->off_scratch);
  p.cnt1 = (unsigned*)(w + L->off_cnt1), p.cnt2 = (unsigned*)(w + L->off_cnt2);
  p.status = (int*)(w + L->off_status);
  p.gridbar = (unsigned*)(w + L->off_status + 64);
  p.debug = (long long*)(w + L->off_debug);
  p.Umax = L->E < M * L->top_k ? L->E : M * L->top_k;
  if (write_tables) {
    p.experts_out = (int*)(w + L->off_tables);
    p.offsets_out = p.experts_out + L->umax_cap;
    p.pairs_out = p.offsets_out + L->umax_cap + 1;
  }
  p.s1_expert_stride = L->s1_stride, p.s2_expert_stride = L->s2_stride;
  p.M = M, p.E = L->E, p.H = L->H, p.I = L->I, p.top_k = L->top_k, p.phases = phases;
  {
    const char* c = getenv("B200MOE_COOPERATIVE");
    p.cooperative = c && c[0] == '1';
  }
  p.KB1 = L->KB1, p.KB2 = L->KB2, p.CB1 = L->CB1, p.NB2 = L->NB2, p.KT1 = L->KT1, p.KT2 = L->KT2;
  const int nb8 = M <= 8 ? 1 : 2;
  const int slab = nb8 * 4096;
  const int limit = 227 * 1024;
  int NS = 8;
  for (; NS >= 2; NS -= 2) {
    const int region = (L->KB1 * slab > NS * slab) ? L->KB1 * slab : NS * slab;
    if (b200_decode_smem_bytes(NS, region) <= limit) { p.region_bytes = region; break; }
  }
  if (NS < 2) return B200MOE_ERR_SHAPE;
  p.NS = NS;
  return b200_decode_launch(p, L->sms, b200_decode_smem_bytes(NS, p.region_bytes), (cudaStream_t)stream);
}

// The whole decode layer: out[M, H] (bf16) = sum_j w[t,j] * FC2_e(silu(gate) * up), e = ids[t,j]. M <= 16.
// Replaces sm120fp4.vllm_backend.Weights._slice (vllm_backend.py:174-190): route + FC1 + FC2 in one launch.
// flags bit 0 (B200MOE_ORDERED): both kernels of the call are ordinary stream-ordered launches.
extern "C" int b200moe_decode_forward_ex(const b200moe_layer* L, const void* x_bf16, const int* topk_ids, const float* topk_weights,
                                         int M, void* out_bf16, void* workspace, long long workspace_bytes, int flags, void* stream) {
  // the tcgen05 kernel whenever the tile records exist and the shape fits it: x scale tiles of <= 12 K boxes in TMEM, one
  // worker group per 128-row output block
  if (L && L->w1t && L->decode_impl != 1 && L->sms <= 256 && L->KB1 <= 12 && L->NB2 <= L->sms) {
    if (!x_bf16 || !topk_ids || !topk_weights || !out_bf16 || !workspace || M < 0) return B200MOE_ERR_ARG;
    if (M > 16) return B200MOE_ERR_LIMIT;
    if (workspace_bytes < L->ws_bytes) return B200MOE_ERR_WORKSPACE;
    if (((uintptr_t)workspace & 255) || ((uintptr_t)x_bf16 & 15)) return B200MOE_ERR_ARG;
    if (M == 0) return B200MOE_OK;
    return decode_tc(const_cast<b200moe_layer*>(L), x_bf16, topk_ids, topk_weights, M, out_bf16, workspace, !(flags & 1), stream);
  }
  return decode_common(L, x_bf16, topk_ids, topk_weights, M, out_bf16, nullptr, 3, 1, workspace, workspace_bytes, stream);
}

extern "C" int b200moe_decode_forward(const b200moe_layer* L, const void* x_bf16, const int* topk_ids, const float* topk_weights,
                                      int M, void* out_bf16, void* workspace, long long workspace_bytes, void* stream) {
  return b200moe_decode_forward_ex(L, x_bf16, topk_ids, topk_weights, M, out_bf16, workspace, workspace_bytes, 0, stream);
}

// The same call for a host that keeps its tensors in host memory. Page-locked buffers (cudaHostAlloc, cudaHostRegister,
// torch's pin_memory) are addressable from the device: the kernels then read x, ids and weights and write the output
// straight across the host link - no copy is enqueued and the transfer overlaps the layer's own work. Pageable buffers are
// copied through staging buffers inside the workspace. Everything is enqueued on `stream`; nothing synchronises.
static void* device_view(const void* host_ptr) {
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, host_ptr) != cudaSuccess) { cudaGetLastError(); return nullptr; }
  if (at.type == cudaMemoryTypeHost || at.type == cudaMemoryTypeManaged || at.type == cudaMemoryTypeDevice) return at.devicePointer;
  return nullptr;
}

extern "C" int b200moe_decode_forward_host(const b200moe_layer* L, const void* x_host, const int* ids_host, const float* wts_host, int M,
                                           void* out_host, void* workspace, long long workspace_bytes, void* stream) {
  if (!L || !x_host || !ids_host || !wts_host || !out_host || !workspace || M < 0) return B200MOE_ERR_ARG;
  if (M > 16) return B200MOE_ERR_LIMIT;
  if (workspace_bytes < L->ws_bytes) return B200MOE_ERR_WORKSPACE;
  if (M == 0) return B200MOE_OK;
  struct DeviceGuard {   // the call may come from a thread whose current device is another one
    int prev = -1;
    explicit DeviceGuard(int want) { if (cudaGetDevice(&prev) == cudaSuccess && prev != want) cudaSetDevice(want); else prev = -1; }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
  } guard(L->device);
  // Page-locked host buffers can be used by the kernels directly across the host link. For the OUTPUT that is a stream of
  // posted writes and saves a copy after the kernel; for the INPUTS it means that all 148 workers fetch the ids and weights
  // from host memory in their prologue, one round trip over the link each, which measures slower than three small copies
  // ahead of the kernel (1.2 TB/s against 0.8 TB/s on the decode sweep). So by default the inputs are staged and the output
  // is written in place; B200MOE_HOST_IN_PLACE=1 uses all four buffers in place, =0 stages all four.
  static const int mode = [] { const char* c = getenv("B200MOE_HOST_IN_PLACE"); return !c ? 2 : c[0] == '0' ? 0 : c[0] == '1' ? 1 : 2; }();
  void* vo = mode != 0 ? device_view(out_host) : nullptr;
  if (mode == 1 && vo) {
    void* vx = device_view(x_host);
    void* vi = device_view(ids_host);
    void* vw = device_view(wts_host);
    if (vx && vi && vw && !((uintptr_t)vx & 15))
      return b200moe_decode_forward(L, vx, (const int*)vi, (const float*)vw, M, vo, workspace, workspace_bytes, stream);
  }
  uint8_t* w = (uint8_t*)workspace;
  cudaStream_t st = (cudaStream_t)stream;
  uint8_t* dx = w + L->off_hstage;
  uint8_t* dout = dx + 16LL * L->H * 2;
  int* dids = (int*)(dout + 16LL * L->H * 2);
  float* dwts = (float*)(dids + 16 * L->top_k);
  B200_CUDA_TRY(cudaMemcpyAsync(dx, x_host, (size_t)M * L->H * 2, cudaMemcpyHostToDevice, st));
  B200_CUDA_TRY(cudaMemcpyAsync(dids, ids_host, (size_t)M * L->top_k * 4, cudaMemcpyHostToDevice, st));
  B200_CUDA_TRY(cudaMemcpyAsync(dwts, wts_host, (size_t)M * L->top_k * 4, cudaMemcpyHostToDevice, st));
  if (vo && !((uintptr_t)vo & 15)) return b200moe_decode_forward(L, dx, dids, dwts, M, vo, workspace, workspace_bytes, stream);
  const int rc = b200moe_decode_forward(L, dx, dids, dwts, M, dout, workspace, workspace_bytes, stream);
  if (rc != B200MOE_OK) return rc;
  B200_CUDA_TRY(cudaMemcpyAsync(out_host, dout, (size_t)M * L->H * 2, cudaMemcpyDeviceToHost, st));
  return B200MOE_OK;
}

// FC1 alone (sm120fp4/kernels/fc1_w4a16.py:251-262, fc1_mma.py:266-282): act[M*top_k, I] bf16, row = pair index.
extern "C" int b200moe_decode_fc1(const b200moe_layer* L, const void* x_bf16, const int* topk_ids, const float* topk_weights, int M,
                                  void* act_bf16, void* workspace, long long workspace_bytes, void* stream) {
  if (!act_bf16) return B200MOE_ERR_ARG;
  return decode_common(L, x_bf16, topk_ids, topk_weights, M, nullptr, act_bf16, 1, 1, workspace, workspace_bytes, stream);
}

// FC2 alone (sm120fp4/kernels/fc2_w4a16.py:276-279, fc2_mma_pf.py:403-421): consumes act[M*top_k, I] bf16.
extern "C" int b200moe_decode_fc2(const b200moe_layer* L, const void* act_bf16, const int* topk_ids, const float* topk_weights, int M,
                                  void* out_bf16, void* workspace, long long workspace_bytes, void* stream) {
  if (!L || !act_bf16 || !topk_ids || !workspace) return B200MOE_ERR_ARG;
  if (M < 0) return B200MOE_ERR_ARG;
  if (M > 16) return B200MOE_ERR_LIMIT;
  if (workspace_bytes < L->ws_bytes) return B200MOE_ERR_WORKSPACE;
  if (M == 0) return B200MOE_OK;
  // routing tables first (phase mask 0 runs only the prologue), then the fragment-ordered copy of the activations
  int rc = decode_common(L, nullptr, topk_ids, topk_weights, M, nullptr, nullptr, 0, 1, workspace, workspace_bytes, stream);
  if (rc != B200MOE_OK) return rc;
  uint8_t* w = (uint8_t*)workspace;
  const int umax = L->E < M * L->top_k ? L->E : M * L->top_k;
  rc = b200_act_to_frag_launch(act_bf16, topk_ids, (const int*)(w + L->off_tables), umax, M, L->top_k, L->I, L->KB2,
                               w + L->off_actfrag, (cudaStream_t)stream);
  if (rc != B200MOE_OK) return rc;
  return decode_common(L, nullptr, topk_ids, topk_weights, M, out_bf16, nullptr, 2, 0, workspace, workspace_bytes, stream);
}

// Copy out the routing tables the last decode call wrote: experts [Umax], offsets [Umax+1], pairs [M*top_k] (device to
// device, on the stream), in the padded form of the reference's GPU router.
extern "C" int b200moe_layer_route_tables(const b200moe_layer* L, const void* workspace, int M, int* experts, int* offsets, int* pairs,
                                          void* stream) {
  if (!L || !workspace || !experts || !offsets || !pairs || M < 0 || M > 16) return B200MOE_ERR_ARG;
  const uint8_t* w = (const uint8_t*)workspace;
  const int umax = L->E < M * L->top_k ? L->E : M * L->top_k;
  const int* t = (const int*)(w + L->off_tables);
  cudaStream_t st = (cudaStream_t)stream;
  B200_CUDA_TRY(cudaMemcpyAsync(experts, t, umax * sizeof(int), cudaMemcpyDeviceToDevice, st));
  B200_CUDA_TRY(cudaMemcpyAsync(offsets, t + L->umax_cap, (umax + 1) * sizeof(int), cudaMemcpyDeviceToDevice, st));
  B200_CUDA_TRY(cudaMemcpyAsync(pairs, t + 2 * L->umax_cap + 1, M * L->top_k * sizeof(int), cudaMemcpyDeviceToDevice, st));
  return B200MOE_OK;
}

// Read the status words (synchronises the stream): 0, or B200MOE_ERR_TIMEOUT (a bounded wait ran out), B200MOE_ERR_ARG
// (expert id out of range), B200MOE_ERR_ORDER (the routing inputs changed under the call), B200MOE_ERR_RANGE (an FC1
// activation beyond the range of the activation scale was clipped). The range and order words are cleared by the read.
static int read_status(const void* workspace, long long off, cudaStream_t st) {
  int w[3] = {0, 0, 0};
  uint8_t* p = (uint8_t*)const_cast<void*>(workspace) + off;
  B200_CUDA_TRY(cudaMemcpyAsync(w, p, sizeof(w), cudaMemcpyDeviceToHost, st));
  B200_CUDA_TRY(cudaStreamSynchronize(st));
  if (w[1] || w[2]) B200_CUDA_TRY(cudaMemsetAsync(p + 4, 0, 8, st));
  if (w[0]) return w[0] == 4 ? B200MOE_ERR_ARG : B200MOE_ERR_TIMEOUT;
  if (w[2]) return B200MOE_ERR_ORDER;
  if (w[1]) return B200MOE_ERR_RANGE;
  return B200MOE_OK;
}

extern "C" int b200moe_layer_status(const b200moe_layer* L, const void* workspace, void* stream) {
  if (!L || !workspace) return B200MOE_ERR_ARG;
  return read_status(workspace, L->off_status, (cudaStream_t)stream);
}

#ifdef B200_DIAGNOSTICS
// Copy the per-worker cycle counters of the last launch to the host (8 int64 per worker, 2 x SM-count workers). Only a
// library built with -DB200_TIMERS fills them; otherwise they read zero. Synchronises the stream.
extern "C" int b200moe_layer_debug_counters(const b200moe_layer* L, const void* workspace, long long* out, int max_workers, void* stream) {
  if (!L || !workspace || !out) return B200MOE_ERR_ARG;
  const int n = 2 * L->sms < max_workers ? 2 * L->sms : max_workers;
  B200_CUDA_TRY(cudaMemcpyAsync(out, (const uint8_t*)workspace + L->off_debug, (size_t)n * 128, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  B200_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  return n;
}
#endif  // B200_DIAGNOSTICS

// ---- W4A4 prefill (any number of tokens up to the workspace's max_tokens): own tcgen05 grouped GEMM, replacing the
// third-party CUTLASS hand-off of sm120fp4/vllm_backend.py:123-168. Needs b200moe_layer_prepack (weight tile records).
long long b200_prefill_workspace_bytes(int E, int H, int I, int top_k, int max_tokens);
int b200_prefill_forward(int E, int H, int I, int top_k, const uint8_t* w1t, const uint8_t* w2t, const float* alpha1, const float* alpha2,
                         const void* x, const int* ids, const float* wts, int M, void* out, void* ws, long long ws_bytes, int ws_tokens,
                         float gs_x, float gs_a, int sms, cudaStream_t st);
int b200_prefill_status_offset(int E, int H, int I, int top_k, int max_tokens, long long* off);
void b200_prefill_workspace_map(int E, int H, int I, int top_k, int max_tokens, long long* out);

extern "C" long long b200moe_prefill_workspace_bytes(const b200moe_layer* L, int max_tokens) {
  if (!L || max_tokens <= 0) return B200MOE_ERR_ARG;
  return b200_prefill_workspace_bytes(L->E, L->H, L->I, L->top_k, max_tokens);
}

// x bf16 [M, H], topk_ids i32 [M, top_k], topk_weights f32 [M, top_k] -> out bf16 [M, H]. gs_x / gs_a: global scales of the
// NVFP4 quantisation of x and of the SiLU*mul activations (1 / the checkpoint's input scales; 1.0 reproduces the reference's
// own W4A4 arithmetic). The workspace must have been sized for max_tokens >= M and zeroed once.
extern "C" int b200moe_prefill_forward(const b200moe_layer* L, const void* x_bf16, const int* topk_ids, const float* topk_weights, int M,
                                       void* out_bf16, void* workspace, long long workspace_bytes, int max_tokens, float gs_x, float gs_a,
                                       void* stream) {
  if (!L || !x_bf16 || !topk_ids || !topk_weights || !out_bf16 || !workspace || M < 0 || max_tokens <= 0) return B200MOE_ERR_ARG;
  if (!L->w1t) return B200MOE_ERR_ARG;   // not prepacked
  if (!(gs_x > 0.f) || !(gs_a > 0.f)) return B200MOE_ERR_ARG;
  if (((uintptr_t)workspace & 255) || ((uintptr_t)x_bf16 & 15) || ((uintptr_t)out_bf16 & 15)) return B200MOE_ERR_ARG;
  if (L->H % 128 || L->I % 64) return B200MOE_ERR_SHAPE;
  if (M == 0) return B200MOE_OK;
  return b200_prefill_forward(L->E, L->H, L->I, L->top_k, L->w1t, L->w2t, L->alpha1, L->alpha2, x_bf16, topk_ids, topk_weights, M, out_bf16,
                              workspace, workspace_bytes, max_tokens, gs_x, gs_a, L->sms, (cudaStream_t)stream);
}

// Where the tables and tile records sit inside a prefill workspace sized for max_tokens (14 values, see the header): lets a
// tool or a test read back what each stage of the last call wrote (router tables, NVFP4 records of x and of the SiLU*mul
// activations, weighted rows). Host-side arithmetic only.
extern "C" int b200moe_prefill_workspace_map(const b200moe_layer* L, int max_tokens, long long* out14) {
  if (!L || !out14 || max_tokens <= 0) return B200MOE_ERR_ARG;
  b200_prefill_workspace_map(L->E, L->H, L->I, L->top_k, max_tokens, out14);
  return B200MOE_OK;
}

// status word of the prefill workspace; synchronises the stream
extern "C" int b200moe_prefill_status(const b200moe_layer* L, const void* workspace, int max_tokens, void* stream) {
  if (!L || !workspace) return B200MOE_ERR_ARG;
  long long off = 0;
  b200_prefill_status_offset(L->E, L->H, L->I, L->top_k, max_tokens, &off);
  int st = 0;
  B200_CUDA_TRY(cudaMemcpyAsync(&st, (const uint8_t*)workspace + off, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  B200_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
  return st == 0 ? B200MOE_OK : B200MOE_ERR_TIMEOUT;
}

// ---- W4A16 layer call for mid-sized batches (17 tokens up to a few hundred): the decode kernels' arithmetic as a grouped
// GEMM over per-expert gathered rows, one pass over the touched experts' weights. The reference runs such batches as slices
// of 16 through its decode kernels (sm120fp4/vllm_backend.py:147-172). Needs b200moe_layer_prepack.
long long b200_mid_workspace_bytes(int E, int H, int I, int top_k, int max_tokens);
int b200_mid_status_offset(int E, int H, int I, int top_k, int max_tokens, long long* off);
int b200_mid_forward(int E, int H, int I, int top_k, const uint8_t* w1t, const uint8_t* w2t, const float* alpha1, const float* alpha2,
                     const void* x, const int* ids, const float* wts, int M, void* out, void* ws, long long ws_bytes, int ws_tokens,
                     float act_g1, int sms, cudaStream_t st);

extern "C" long long b200moe_mid_workspace_bytes(const b200moe_layer* L, int max_tokens) {
  if (!L || max_tokens <= 0) return B200MOE_ERR_ARG;
  if (L->KB1 > 12 || L->KB2 > 12) return B200MOE_ERR_SHAPE;   // the operand tile's scale columns (16 per K box) must fit in TMEM
  return b200_mid_workspace_bytes(L->E, L->H, L->I, L->top_k, max_tokens);
}

// x bf16 [M, H], topk_ids i32 [M, top_k], topk_weights f32 [M, top_k] -> out bf16 [M, H]; M <= max_tokens of the (zeroed)
// workspace. Same arithmetic as b200moe_decode_forward (W4A16, fp32 accumulation).
extern "C" int b200moe_mid_forward(const b200moe_layer* L, const void* x_bf16, const int* topk_ids, const float* topk_weights, int M,
                                   void* out_bf16, void* workspace, long long workspace_bytes, int max_tokens, void* stream) {
  if (!L || !x_bf16 || !topk_ids || !topk_weights || !out_bf16 || !workspace || M < 0 || max_tokens <= 0) return B200MOE_ERR_ARG;
  if (!L->w1t) return B200MOE_ERR_ARG;   // not prepacked
  if (((uintptr_t)workspace & 255) || ((uintptr_t)x_bf16 & 15) || ((uintptr_t)out_bf16 & 15)) return B200MOE_ERR_ARG;
  if (L->H % 128 || L->I % 64) return B200MOE_ERR_SHAPE;
  if (M == 0) return B200MOE_OK;
  return b200_mid_forward(L->E, L->H, L->I, L->top_k, L->w1t, L->w2t, L->alpha1, L->alpha2, x_bf16, topk_ids, topk_weights, M, out_bf16,
                          workspace, workspace_bytes, max_tokens, L->act_g1, L->sms, (cudaStream_t)stream);
}

// status word of the mid-batch workspace; synchronises the stream
extern "C" int b200moe_mid_status(const b200moe_layer* L, const void* workspace, int max_tokens, void* stream) {
  if (!L || !workspace) return B200MOE_ERR_ARG;
  long long off = 0;
  b200_mid_status_offset(L->E, L->H, L->I, L->top_k, max_tokens, &off);
  return read_status(workspace, off, (cudaStream_t)stream);
}

extern "C" int b200moe_layer_sm_count(const b200moe_layer* L) { return L ? L->sms : B200MOE_ERR_ARG; }

// Where the tcgen05 decode kernel's operands sit inside a decode workspace, for tools and tests that read back what the last
// call computed with: out8 = offset of the expanded x operand, of its 1/g_t column scales, of the expanded FC1->FC2
// activation slabs, bytes of one slab for N = 16 / 32 / 64 operand columns, the first-term activation scale as float bits,
// and the capacity (touched experts) of the slab array.
extern "C" int b200moe_layer_workspace_map(const b200moe_layer* L, long long* out8) {
  if (!L || !out8) return B200MOE_ERR_ARG;
  out8[0] = L->off_xb, out8[1] = L->off_xscale, out8[2] = L->off_aslab;
  out8[3] = 16 * 128 + 2048, out8[4] = 32 * 128 + 2048, out8[5] = 64 * 128 + 2048;
  unsigned bits;
  memcpy(&bits, &L->act_g1, 4);
  out8[6] = bits, out8[7] = L->umax_cap;
  return B200MOE_OK;
}
