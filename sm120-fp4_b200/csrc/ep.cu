// Expert-parallel dispatch and combine for the fixed-capacity exchange (decode batches): two small kernels around the
// NCCL all-to-all, replacing a dozen framework element-wise launches. The reference has no expert parallelism (its
// `fits()` declines `use_ep`, sm120fp4/vllm_classes.py:46-47), so these entry points have no counterpart there.
#include "common.cuh"
#include "ptx.cuh"
#include <cuda_bf16.h>
#include <stdint.h>
#include <string.h>

namespace b200 {

// Block (row, dest): row `row` of the block sent to rank `dest` is token `row` (zeros beyond the batch), its top-k slots
// re-indexed to the destination's local experts; slots the destination does not own become id -1 / weight 0.
// Where a block lands is given per destination: D.x[dest] / D.ids[dest] / D.wts[dest] point at the block's rows, local ids
// and weights (cap rows each). For the NCCL exchange they point into one packed send buffer (rows | ids | weights per
// destination, so that ONE all-to-all carries all three); for the peer-store exchange they point straight into the
// destination GPU's receive arrays across NVLink (plain stores; no multicast), and D.flag[dest] is a counter in the
// destination's memory that every block bumps (system-scope, after a system-scope fence) once its row has been stored.
constexpr int kEpMaxWorld = 16;
// Kernels whose blocks wait for a peer's words or counters need every block of their grid (cap x world blocks of 128 threads)
// resident at once, on every rank: a waiting block that keeps the block it waits for (on the peer) from being scheduled
// would only end by its bounded wait. 1024 blocks fit beside a layer kernel on any B200; the peer-store exchange is for
// decode-sized blocks, larger ones go through the stream-ordered exchange.
constexpr int kEpMaxWaitingBlocks = 1024;

struct EpDest {
  __nv_bfloat16* x[kEpMaxWorld];
  int* ids[kEpMaxWorld];
  float* wts[kEpMaxWorld];
  unsigned* flag[kEpMaxWorld];   // null: no signalling (stream-ordered exchange follows)
};

// Bounded wait on `world` arrival counters (lane s polls counter s) until each has reached `want`; a wait that runs out sets
// *status to 1 + the late peer's rank and returns. Called by one whole warp.
__device__ __forceinline__ void ep_wait_counters(const unsigned* flags, int world, unsigned want, int* status) {
  const int s = threadIdx.x & 31;
  if (s < world) {
    bool ok = false;
    for (unsigned it = 0; it < (1u << 22); ++it) {
      unsigned v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + s) : "memory");
      if ((int)(v - want) >= 0) { ok = true; break; }
      if (it > 1024u) __nanosleep(200);
    }
    if (!ok) *status = 1 + s;
  }
  __syncwarp();
}

struct EpWait {
  const unsigned* flags;   // null: the kernel does not wait
  unsigned* calls;         // this rank's call counter (only ever incremented, once per layer call, by the dispatch kernel)
  int* status;
  int world;
  unsigned per_call;
};

__global__ void __launch_bounds__(128) k_ep_dispatch(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids,
                                                     const float* __restrict__ wts, int m, int h, int k, int per, const __grid_constant__ EpDest D,
                                                     const EpWait W) {
  const int row = blockIdx.x, dest = blockIdx.y;
  uint4* dst = reinterpret_cast<uint4*>(D.x[dest] + (long long)row * h);
  const uint4* src = reinterpret_cast<const uint4*>(x + (long long)row * h);
  bool any = false;
  if (row < m)
    for (int j = 0; j < k; ++j) { const int e = ids[row * k + j]; any |= e >= 0 && e / per == dest; }
  // a row none of whose experts live on the destination travels as its (all empty) slots only: the kernels skip such rows
  if (any) for (int i = threadIdx.x; i < h / 8; i += blockDim.x) dst[i] = src[i];
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    int id = -1;
    float w = 0.f;
    if (row < m) {
      const int e = ids[row * k + j];
      if (e >= 0 && e / per == dest) { id = e - dest * per; w = wts[row * k + j]; }
    }
    D.ids[dest][row * k + j] = id;
    D.wts[dest][row * k + j] = w;
  }
  if (D.flag[dest]) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      atomicAdd_system(D.flag[dest], 1u);
    }
  }
  // Peer-store exchange: the kernel only completes when every peer's rows of this call have arrived (one block waits; the
  // peers' sends do not depend on this wait), so whatever follows in the stream finds its input in place.
  if (W.flags && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < 32) {
    const unsigned n = W.calls[0] + 1u;
    ep_wait_counters(W.flags, W.world, n * W.per_call, W.status);
    if (threadIdx.x == 0) W.calls[0] = n;
  }
}

// Bounded wait of the consumer side of the peer-store exchange: thread s waits until peer s has bumped flags[s] `per_call`
// more times than this rank has consumed so far (calls[0] counts this rank's calls; the counters only ever grow, so nothing is
// reset between calls). A wait that runs out sets *status and returns - the data of that peer is then stale, which the
// caller learns from the status word, not from a hang.
__global__ void k_ep_wait(const unsigned* __restrict__ flags, int world, unsigned per_call, unsigned* __restrict__ calls, int* __restrict__ status) {
  const unsigned want = (calls[0] + 1u) * per_call;
  ep_wait_counters(flags, world, want, status);
  if (threadIdx.x == 0) calls[0] += 1u;
}

// Received blocks of the NCCL exchange (per source: rows | ids | weights) -> the contiguous arrays the layer call takes.
__global__ void __launch_bounds__(128) k_ep_unpack(const uint8_t* __restrict__ rbuf, long long block_bytes, int cap, int h, int k,
                                                   __nv_bfloat16* __restrict__ rx, int* __restrict__ rid, float* __restrict__ rw) {
  const int row = blockIdx.x, srcr = blockIdx.y;
  const uint8_t* blk = rbuf + srcr * block_bytes;
  const int* bid = reinterpret_cast<const int*>(blk + (long long)cap * h * 2) + row * k;
  const float* bw = reinterpret_cast<const float*>(blk + (long long)cap * h * 2 + (long long)cap * k * 4) + row * k;
  const long long o = (long long)srcr * cap + row;
  bool any = false;
  for (int j = 0; j < k; ++j) any |= bid[j] >= 0;
  if (any) {
    const uint4* src = reinterpret_cast<const uint4*>(blk + (long long)row * h * 2);
    uint4* dst = reinterpret_cast<uint4*>(rx + o * h);
    for (int i = threadIdx.x; i < h / 8; i += blockDim.x) dst[i] = src[i];
  }
  for (int j = threadIdx.x; j < k; j += blockDim.x) { rid[o * k + j] = bid[j]; rw[o * k + j] = bw[j]; }
}

// The partial rows a rank computed for source s (rows s*cap .. s*cap + cap of yl) go back into s's `back` array at block
// `rank` by plain peer stores, then one bump of s's return flag per row.
struct EpBack {
  __nv_bfloat16* y[kEpMaxWorld];
  unsigned* flag[kEpMaxWorld];
};

// With `out` the same kernel also finishes the layer call: block (row, 0) then waits (bounded) until every peer's partial
// rows of this call are in this rank's `back` array and writes out[row] = bf16(sum over ranks, in rank order, in fp32).
__global__ void __launch_bounds__(128) k_ep_return(const __nv_bfloat16* __restrict__ yl, int cap, int h, int rank, const __grid_constant__ EpBack B,
                                                   const EpWait W, const __nv_bfloat16* __restrict__ back, int m, int world,
                                                   __nv_bfloat16* __restrict__ out) {
  const int row = blockIdx.x, srcr = blockIdx.y;
  const uint4* src = reinterpret_cast<const uint4*>(yl + ((long long)srcr * cap + row) * h);
  uint4* dst = reinterpret_cast<uint4*>(B.y[srcr] + ((long long)rank * cap + row) * h);
  for (int i = threadIdx.x; i < h / 8; i += blockDim.x) dst[i] = src[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    atomicAdd_system(B.flag[srcr], 1u);
  }
  if (!out || srcr != 0 || row >= m) return;
  if (threadIdx.x < 32) ep_wait_counters(W.flags, W.world, W.calls[0] * W.per_call, W.status);   // the dispatch kernel of this call counted it
  __syncthreads();
  for (int c = threadIdx.x; c < h / 8; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(back + ((long long)r * cap + row) * h + c * 8));
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += __uint_as_float(w4[q] << 16);
        acc[2 * q + 1] += __uint_as_float(w4[q] & 0xffff0000u);
      }
    }
    uint32_t o4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat162 hh = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      o4[q] = *reinterpret_cast<const uint32_t*>(&hh);
    }
    *reinterpret_cast<uint4*>(out + (long long)row * h + c * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
  }
}

// out[t] = bf16( sum over ranks r = 0..world-1, in that order, of float(y[r][t]) ): bit-identical from call to call.
__global__ void __launch_bounds__(256) k_ep_combine(const __nv_bfloat16* __restrict__ y, int m, int h, int world, int cap,
                                                    __nv_bfloat16* __restrict__ out) {
  const int chunks = h / 8;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < m * chunks; i += gridDim.x * blockDim.x) {
    const int t = i / chunks, c = i - t * chunks;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < world; ++r) {
      const uint4 v = *reinterpret_cast<const uint4*>(y + ((long long)r * cap + t) * h + c * 8);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += __uint_as_float(w4[q] << 16);
        acc[2 * q + 1] += __uint_as_float(w4[q] & 0xffff0000u);
      }
    }
    uint32_t o4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat162 hh = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      o4[q] = *reinterpret_cast<const uint32_t*>(&hh);
    }
    *reinterpret_cast<uint4*>(out + (long long)t * h + c * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// The peer-store exchange without a fence: every 8-byte store carries 4 bytes of payload and the call number ("flagged
// words", the low-latency protocol of collective libraries). An aligned 8-byte store arrives whole, so a receiver that sees
// the current call number in a word has that word's payload; nothing has to order the payload before a separate flag, i.e.
// the sender never waits for its stores to be acknowledged across NVLink (a system-scope fence there costs a round trip,
// 2-3 us, in each of the two exchanges of a layer call). The price is twice the bytes (8 KB per 4 KB row), which is
// nothing at decode sizes. Buffers are zeroed once; call numbers start at 1 and only grow, so a stale word never matches.
//
// Flagged row of the dispatch: h/2 words of x (two bf16 each), then k words of local expert ids, then k words of routing
// weights. A row whose token has no expert on the destination travels as its 2k meta words only.
struct EpLLPeers {
  uint2* p[kEpMaxWorld];   // per peer: where THIS rank's block starts in the peer's flagged receive area
};

__device__ __forceinline__ void ll_store(uint2* dst, uint32_t payload, uint32_t flag) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(payload), "r"(flag) : "memory");
}

// Flagged words in batches: up to kLLBatch words per thread are read (or written) back to back, so their latencies overlap
// instead of adding up (a thread that polls its words one after the other pays an L2 round trip for each).
constexpr int kLLBatch = 8;

// src[i] -> flagged words dst[i] for i = first, first + stride, ... < count
__device__ __forceinline__ void ll_send(uint2* dst, const uint32_t* __restrict__ src, int first, int stride, int count, uint32_t flag) {
  for (int b0 = first; b0 < count; b0 += stride * kLLBatch) {
    uint32_t v[kLLBatch];
#pragma unroll
    for (int j = 0; j < kLLBatch; ++j) v[j] = b0 + j * stride < count ? src[b0 + j * stride] : 0u;
#pragma unroll
    for (int j = 0; j < kLLBatch; ++j)
      if (b0 + j * stride < count) ll_store(dst + b0 + j * stride, v[j], flag);
  }
}

// Bounded poll of the flagged words src[i], i = b0 + j * stride (j < kLLBatch, i < count): payloads into v[]; false (and
// *status = 1 + peer) when the call number never shows up in one of them.
__device__ __forceinline__ bool ll_recv_batch(const uint2* src, int b0, int stride, int count, uint32_t flag, uint32_t* v, int peer, int* status) {
  unsigned pending = 0;
#pragma unroll
  for (int j = 0; j < kLLBatch; ++j)
    if (b0 + j * stride < count) pending |= 1u << j;
  for (unsigned it = 0; it < (1u << 22); ++it) {
    uint32_t a[kLLBatch], f[kLLBatch];
#pragma unroll
    for (int j = 0; j < kLLBatch; ++j)
      if ((pending >> j) & 1u)
        asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(a[j]), "=r"(f[j]) : "l"(src + b0 + j * stride) : "memory");
#pragma unroll
    for (int j = 0; j < kLLBatch; ++j)
      if (((pending >> j) & 1u) && f[j] == flag) { v[j] = a[j]; pending &= ~(1u << j); }
    if (!pending) return true;
    if (it > 2048u) __nanosleep(200);
    if ((it & 1023u) == 1023u && *reinterpret_cast<volatile int*>(status) != 0) return false;   // another wait already gave up
  }
  *status = 1 + peer;
  return false;
}

// Bounded poll of one flagged word; false (and *status = 1 + peer) when the call number never shows up.
__device__ __forceinline__ bool ll_load(const uint2* src, uint32_t flag, uint32_t* payload, int peer, int* status) {
  for (unsigned it = 0; it < (1u << 22); ++it) {
    uint32_t a, b;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "l"(src) : "memory");
    if (b == flag) { *payload = a; return true; }
    if (it > 2048u) __nanosleep(200);
    if ((it & 1023u) == 1023u && *reinterpret_cast<volatile int*>(status) != 0) return false;   // another wait already gave up
  }
  *status = 1 + peer;
  return false;
}

// Dispatch and receive in one launch. Block (row, peer): first it sends token `row` to `peer` (flagged words into the peer's
// receive area), then it receives row `row` of `peer`'s block from this rank's own receive area `in` ([world][cap][words])
// into the plain arrays the layer call takes (rx bf16 [world * cap, h], rid int32 / rw f32 [world * cap, k]). calls[0] is
// the number of completed layer calls (read here, advanced by the return kernel); calls[1] is advanced here for the return
// kernel to read - neither kernel reads the word it writes, so the blocks of a launch agree on the call number.
__global__ void __launch_bounds__(128) k_ep_dispatch_ll(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids,
                                                        const float* __restrict__ wts, int m, int h, int k, int per, int cap,
                                                        const __grid_constant__ EpLLPeers D, const uint2* __restrict__ in,
                                                        __nv_bfloat16* __restrict__ rx, int* __restrict__ rid, float* __restrict__ rw,
                                                        unsigned* __restrict__ calls, int* __restrict__ status) {
  const int row = blockIdx.x, peer = blockIdx.y, tid = threadIdx.x;
  const uint32_t n = calls[0] + 1u;
  const int hw = h / 2, words = hw + 2 * k;
  // ---- send
  {
    uint2* dst = D.p[peer] + (long long)row * words;
    bool any = false;
    if (row < m)
      for (int j = 0; j < k; ++j) { const int e = ids[row * k + j]; any |= e >= 0 && e / per == peer; }
    if (tid < 2 * k) {
      const int j = tid < k ? tid : tid - k;
      int id = -1;
      float w = 0.f;
      if (row < m) {
        const int e = ids[row * k + j];
        if (e >= 0 && e / per == peer) { id = e - peer * per; w = wts[row * k + j]; }
      }
      ll_store(dst + hw + tid, tid < k ? (uint32_t)id : __float_as_uint(w), n);
    }
    if (any) ll_send(dst, reinterpret_cast<const uint32_t*>(x + (long long)row * h), tid, (int)blockDim.x, hw, n);
  }
  // ---- receive
  {
    const uint2* src = in + ((long long)peer * cap + row) * words;
    const long long o = (long long)peer * cap + row;
    int id = -1;
    bool ok = true;
    if (tid < 2 * k) {
      uint32_t v = 0;
      ok = ll_load(src + hw + tid, n, &v, peer, status);
      if (tid < k) { id = ok ? (int)v : -1; rid[o * k + tid] = id; }
      else rw[o * k + tid - k] = ok ? __uint_as_float(v) : 0.f;
      __threadfence();
    }
    const int any = __syncthreads_or(tid < k && id >= 0);
    // The ids and weights of this block's row are in place: a layer kernel launched programmatically behind this one may
    // start once every block is this far - it reads them in its prologue (and checks them again after the stream dependency
    // has resolved), builds its routing tables and starts streaming weights while the rows themselves are still arriving;
    // it waits for this kernel to complete before it touches a row.
    grid_launch_dependents();
    if (any) {
      uint32_t* dst = reinterpret_cast<uint32_t*>(rx + o * h);
      const int stride = (int)blockDim.x;
      for (int b0 = tid; b0 < hw; b0 += stride * kLLBatch) {
        uint32_t v[kLLBatch];
        if (!ll_recv_batch(src, b0, stride, hw, n, v, peer, status)) break;
#pragma unroll
        for (int j = 0; j < kLLBatch; ++j)
          if (b0 + j * stride < hw) dst[b0 + j * stride] = v[j];
      }
    }
  }
  if (blockIdx.x == 0 && blockIdx.y == 0 && tid == 0) calls[1] = n;
}

// Return, receive and combine in one launch. Block (row, peer): if this rank computed anything for token `row` of `peer`
// (one of the row's received ids is live), its partial row goes back as flagged words into `peer`'s return area at block
// `rank`. Blocks (row, 0) with row < m then finish the layer call for token `row`: for every rank r in rank order that owns
// one of the token's experts they take r's flagged partial row from this rank's own return area `back` ([world][cap][h/2])
// and add it in fp32; one bf16 rounding. Ranks that own none of the token's experts sent nothing and are not waited for.
// Return area of a rank: uint2 [world][cap][h/2] rows, then `world` marker words.
__global__ void __launch_bounds__(128) k_ep_return_ll(const __nv_bfloat16* __restrict__ yl, const int* __restrict__ rid, int cap, int h, int k,
                                                      int rank, int world, int per, const __grid_constant__ EpLLPeers B,
                                                      const uint2* __restrict__ back, const int* __restrict__ ids, int m,
                                                      __nv_bfloat16* __restrict__ out, unsigned* __restrict__ calls, int* __restrict__ status) {
  const int row = blockIdx.x, peer = blockIdx.y, tid = threadIdx.x;
  grid_dependency_wait();   // launched programmatically behind the layer kernel (its launch latency hidden): yl is complete from here on
  const uint32_t n = calls[1];
  const int hw = h / 2;
  const long long marks = (long long)world * cap * hw;   // after the rows of a return area: one word per rank, "rank r has reached its return of call n"
  if (row == 0 && tid == 0) ll_store(B.p[peer] - (long long)rank * cap * hw + marks + rank, 0u, n);
  {
    const long long o = (long long)peer * cap + row;
    bool any = false;
    for (int j = 0; j < k; ++j) any |= rid[o * k + j] >= 0;
    if (any) {
      ll_send(B.p[peer] + (long long)row * hw, reinterpret_cast<const uint32_t*>(yl + o * h), tid, (int)blockDim.x, hw, n);
    }
  }
  if (peer == 0 && row < m) {
    unsigned owners = 0;   // bit r: rank r owns one of this token's experts and returns a partial row
    for (int j = 0; j < k; ++j) {
      const int e = ids[row * k + j];
      if (e >= 0 && e / per < world) owners |= 1u << (e / per);
    }
    const int stride = (int)blockDim.x;
    for (int b0 = tid; b0 < hw; b0 += stride * kLLBatch) {
      float a0[kLLBatch], a1[kLLBatch];
#pragma unroll
      for (int j = 0; j < kLLBatch; ++j) a0[j] = a1[j] = 0.f;
      bool ok = true;
      for (int r = 0; r < world && ok; ++r) {
        if (!((owners >> r) & 1u)) continue;
        uint32_t v[kLLBatch];
        ok = ll_recv_batch(back + ((long long)r * cap + row) * hw, b0, stride, hw, n, v, r, status);
#pragma unroll
        for (int j = 0; j < kLLBatch; ++j)
          if (ok && b0 + j * stride < hw) {
            a0[j] += __uint_as_float(v[j] << 16);
            a1[j] += __uint_as_float(v[j] & 0xffff0000u);
          }
      }
      if (!ok) break;
#pragma unroll
      for (int j = 0; j < kLLBatch; ++j)
        if (b0 + j * stride < hw) {
          const __nv_bfloat162 hh = __floats2bfloat162_rn(a0[j], a1[j]);
          reinterpret_cast<uint32_t*>(out + (long long)row * h)[b0 + j * stride] = *reinterpret_cast<const uint32_t*>(&hh);
        }
    }
  }
  // The call is complete on this rank once every rank has reached its own return kernel: from then on no peer reads this
  // call's words of this rank any more, so the next call's words may overwrite them. (The row waits above skip the ranks
  // that own none of a token's experts, so they alone would not order this rank behind all the others.)
  if (blockIdx.x == 0 && blockIdx.y == 0 && tid < 32) {
    uint32_t v;
    if (tid < world) ll_load(back + marks + tid, n, &v, tid, status);
    __syncwarp();
    if (tid == 0) calls[0] = n;
  }
}

}  // namespace b200

using namespace b200;

// x bf16 [m, h], ids int32 [m, k] (global expert ids, negative = empty slot), wts f32 [m, k] -> per destination d a block of
// cap rows: rows at dst_x[d] (bf16 [cap, h]), local ids at dst_ids[d] (int32 [cap, k]), weights at dst_wts[d] (f32 [cap, k]);
// the three pointer tables are HOST arrays of `world` device pointers. dst_flag: null, or a host array of `world` device
// pointers to counters that every block bumps after its row is stored (peer-store exchange). experts_per_rank = E / world;
// m <= cap; h a multiple of 8. A row is copied only where the destination owns one of its experts.
static int ep_dispatch(const void* x, const int* ids, const float* wts, int m, int h, int k, int world, int experts_per_rank, int cap,
                       void* const* dst_x, int* const* dst_ids, float* const* dst_wts, unsigned* const* dst_flag, const EpWait& W, void* stream) {
  if (!x || !ids || !wts || !dst_x || !dst_ids || !dst_wts) return B200MOE_ERR_ARG;
  if (m < 0 || m > cap || h <= 0 || h % 8 || k < 1 || world < 1 || world > kEpMaxWorld || experts_per_rank < 1 || cap < 1) return B200MOE_ERR_SHAPE;
  EpDest D;
  for (int d = 0; d < kEpMaxWorld; ++d) {
    const bool live = d < world;
    D.x[d] = live ? (__nv_bfloat16*)dst_x[d] : nullptr;
    D.ids[d] = live ? dst_ids[d] : nullptr;
    D.wts[d] = live ? dst_wts[d] : nullptr;
    D.flag[d] = live && dst_flag ? dst_flag[d] : nullptr;
    if (live && (!D.x[d] || !D.ids[d] || !D.wts[d])) return B200MOE_ERR_ARG;
  }
  k_ep_dispatch<<<dim3(cap, world), 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ids, wts, m, h, k, experts_per_rank, D, W);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

extern "C" int b200moe_ep_dispatch(const void* x, const int* ids, const float* wts, int m, int h, int k, int world, int experts_per_rank,
                                   int cap, void* const* dst_x, int* const* dst_ids, float* const* dst_wts, unsigned* const* dst_flag,
                                   void* stream) {
  const EpWait none = {nullptr, nullptr, nullptr, 0, 0u};
  return ep_dispatch(x, ids, wts, m, h, k, world, experts_per_rank, cap, dst_x, dst_ids, dst_wts, dst_flag, none, stream);
}

// The peer-store dispatch and the wait for the peers' rows in ONE launch: as b200moe_ep_dispatch with dst_flag, and the kernel
// only completes once the counters in `flags_in` (this rank's, one per peer) have all grown by `cap` since the previous
// call; `calls` (device, zeroed once) counts this rank's calls.
extern "C" int b200moe_ep_dispatch_wait(const void* x, const int* ids, const float* wts, int m, int h, int k, int world, int experts_per_rank,
                                        int cap, void* const* dst_x, int* const* dst_ids, float* const* dst_wts, unsigned* const* dst_flag,
                                        const unsigned* flags_in, unsigned* calls, int* status, void* stream) {
  if (!dst_flag || !flags_in || !calls || !status) return B200MOE_ERR_ARG;
  const EpWait W = {flags_in, calls, status, world, (unsigned)cap};
  return ep_dispatch(x, ids, wts, m, h, k, world, experts_per_rank, cap, dst_x, dst_ids, dst_wts, dst_flag, W, stream);
}

// rbuf: `world` received blocks of block_bytes each (rows bf16 [cap, h] | ids int32 [cap, k] | weights f32 [cap, k]) ->
// rx bf16 [world * cap, h], rid int32 [world * cap, k], rw f32 [world * cap, k]
extern "C" int b200moe_ep_unpack(const void* rbuf, long long block_bytes, int world, int cap, int h, int k, void* rx, int* rid, float* rw,
                                 void* stream) {
  if (!rbuf || !rx || !rid || !rw) return B200MOE_ERR_ARG;
  if (world < 1 || cap < 1 || h <= 0 || h % 8 || k < 1 || block_bytes < (long long)cap * (h * 2 + k * 8) || block_bytes % 16) return B200MOE_ERR_SHAPE;
  k_ep_unpack<<<dim3(cap, world), 128, 0, (cudaStream_t)stream>>>((const uint8_t*)rbuf, block_bytes, cap, h, k, (__nv_bfloat16*)rx, rid, rw);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// Consumer side of the peer-store exchange: wait (bounded) until every one of `world` peers has bumped its counter in `flags`
// per_call more times; `calls` is this rank's own call counter (device, starts at 0), `status` a device word that a wait that
// ran out sets to 1 + the peer's rank.
extern "C" int b200moe_ep_wait(const unsigned* flags, int world, int per_call, unsigned* calls, int* status, void* stream) {
  if (!flags || !calls || !status) return B200MOE_ERR_ARG;
  if (world < 1 || world > kEpMaxWorld || per_call < 1) return B200MOE_ERR_SHAPE;
  k_ep_wait<<<1, 32, 0, (cudaStream_t)stream>>>(flags, world, (unsigned)per_call, calls, status);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// yl bf16 [world * cap, h] (this rank's partial rows, block s for source s) -> peer s's back array at block `rank`
// (back_y[s]: bf16 [world, cap, h] in s's memory), then cap bumps of back_flag[s]. Host arrays of `world` device pointers.
static int ep_return(const void* yl, int world, int cap, int h, int rank, void* const* back_y, unsigned* const* back_flag, const EpWait& W,
                     const void* back, int m, void* out, void* stream) {
  if (!yl || !back_y || !back_flag) return B200MOE_ERR_ARG;
  if (world < 1 || world > kEpMaxWorld || cap < 1 || h <= 0 || h % 8 || rank < 0 || rank >= world || m < 0 || m > cap) return B200MOE_ERR_SHAPE;
  EpBack B;
  for (int d = 0; d < kEpMaxWorld; ++d) {
    B.y[d] = d < world ? (__nv_bfloat16*)back_y[d] : nullptr;
    B.flag[d] = d < world ? back_flag[d] : nullptr;
    if (d < world && (!B.y[d] || !B.flag[d])) return B200MOE_ERR_ARG;
  }
  k_ep_return<<<dim3(cap, world), 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)yl, cap, h, rank, B, W, (const __nv_bfloat16*)back, m, world,
                                                                  (__nv_bfloat16*)out);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

extern "C" int b200moe_ep_return(const void* yl, int world, int cap, int h, int rank, void* const* back_y, unsigned* const* back_flag,
                                 void* stream) {
  const EpWait none = {nullptr, nullptr, nullptr, 0, 0u};
  return ep_return(yl, world, cap, h, rank, back_y, back_flag, none, nullptr, 0, nullptr, stream);
}

// Return, wait and combine in ONE launch (after b200moe_ep_dispatch_wait of the same call, which counted it in `calls`): the
// partial rows go to their sources; then, per token row, the kernel waits until `flags_back` shows every peer's rows of this
// call in `back` (this rank's bf16 [world, cap, h]) and writes out bf16 [m, h], summed in rank order in fp32.
extern "C" int b200moe_ep_return_combine(const void* yl, int world, int cap, int h, int rank, void* const* back_y, unsigned* const* back_flag,
                                         const unsigned* flags_back, const unsigned* calls, int* status, const void* back, int m, void* out,
                                         void* stream) {
  if (!flags_back || !calls || !status || !back || !out) return B200MOE_ERR_ARG;
  if ((long long)cap * world > kEpMaxWaitingBlocks) return B200MOE_ERR_LIMIT;   // its combining blocks wait for the peers' blocks
  const EpWait W = {flags_back, const_cast<unsigned*>(calls), status, world, (unsigned)cap};
  return ep_return(yl, world, cap, h, rank, back_y, back_flag, W, back, m, out, stream);
}

// y bf16 [world, cap, h] (the partial rows that came back, block r from rank r) -> out bf16 [m, h]
extern "C" int b200moe_ep_combine(const void* y, int m, int h, int world, int cap, void* out, void* stream) {
  if (!y || !out) return B200MOE_ERR_ARG;
  if (m < 0 || m > cap || h <= 0 || h % 8 || world < 1) return B200MOE_ERR_SHAPE;
  if (m == 0) return B200MOE_OK;
  const int total = m * (h / 8);
  k_ep_combine<<<(total + 255) / 256, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)y, m, h, world, cap, (__nv_bfloat16*)out);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// Variable-size exchange (prefill batches): a token row travels once to every rank that owns at least one of its experts.
namespace b200 {

// One block. Thread i owns the contiguous tokens [i*c, (i+1)*c): per destination, an exclusive scan over the threads gives
// every sent (token, destination) its row in the send buffer - destination-major, token order within a destination.
// counts[d] rows go to rank d, offsets[d] is the first of them (offsets[world] = total), pos[t*world + d] the row of token
// t for destination d or -1, send_tok[row] = t.
__global__ void __launch_bounds__(1024) k_ep_plan(const int* __restrict__ ids, int m, int k, int world, int per, int* __restrict__ counts,
                                                  int* __restrict__ offsets, int* __restrict__ pos, int* __restrict__ send_tok) {
  __shared__ int wsum[32];
  __shared__ int s_off[kEpMaxWorld + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c = (m + 1023) / 1024;
  const int t0 = tid * c, t1 = min(m, t0 + c);
  // pass 1: rows per destination
  int running = 0;
  for (int d = 0; d < world; ++d) {
    int mine = 0;
    for (int t = t0; t < t1; ++t) {
      bool hit = false;
      for (int j = 0; j < k; ++j) { const int e = ids[t * k + j]; hit |= e >= 0 && e / per == d; }
      mine += hit;
    }
    int inc = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) { const int a = __shfl_up_sync(0xffffffffu, inc, o); if (lane >= o) inc += a; }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    int base = inc - mine;
    for (int w2 = 0; w2 < warp; ++w2) base += wsum[w2];
    int total = 0;
    for (int w2 = 0; w2 < 32; ++w2) total += wsum[w2];
    if (tid == 0) { s_off[d] = running; counts[d] = total; offsets[d] = running; }
    // pass 2 for this destination: rows of this thread's tokens
    int r = running + base;
    for (int t = t0; t < t1; ++t) {
      bool hit = false;
      for (int j = 0; j < k; ++j) { const int e = ids[t * k + j]; hit |= e >= 0 && e / per == d; }
      pos[t * world + d] = hit ? r : -1;
      if (hit) { send_tok[r] = t; ++r; }
    }
    running += total;
    __syncthreads();
  }
  if (tid == 0) offsets[world] = running;
}

// Block r (< offsets[world]): row r of the send buffer = token send_tok[r] for the destination whose range holds r.
__global__ void __launch_bounds__(128) k_ep_gather(const __nv_bfloat16* __restrict__ x, const int* __restrict__ ids, const float* __restrict__ wts,
                                                   const int* __restrict__ send_tok, const int* __restrict__ offsets, int h, int k, int world,
                                                   int per, __nv_bfloat16* __restrict__ sx, int* __restrict__ meta) {
  for (int r = blockIdx.x; r < offsets[world]; r += gridDim.x) {
    int d = 0;
    while (d + 1 < world && r >= offsets[d + 1]) ++d;
    const int t = send_tok[r];
    const uint4* src = reinterpret_cast<const uint4*>(x + (long long)t * h);
    uint4* dst = reinterpret_cast<uint4*>(sx + (long long)r * h);
    for (int i = threadIdx.x; i < h / 8; i += blockDim.x) dst[i] = src[i];
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
      const int e = ids[t * k + j];
      const bool own = e >= 0 && e / per == d;
      meta[(long long)r * 2 * k + j] = own ? e - d * per : -1;
      meta[(long long)r * 2 * k + k + j] = __float_as_int(own ? wts[t * k + j] : 0.f);
    }
  }
}

// out[t] = bf16( sum over destinations d = 0..world-1, in that order, of float(back[pos[t, d]]) where pos >= 0 )
__global__ void __launch_bounds__(256) k_ep_combine_rows(const __nv_bfloat16* __restrict__ back, const int* __restrict__ pos, int m, int h, int world,
                                                         __nv_bfloat16* __restrict__ out) {
  const int chunks = h / 8;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < m * chunks; i += gridDim.x * blockDim.x) {
    const int t = i / chunks, c = i - t * chunks;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int d = 0; d < world; ++d) {
      const int r = pos[t * world + d];
      if (r < 0) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(back + (long long)r * h + c * 8);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        acc[2 * q] += __uint_as_float(w4[q] << 16);
        acc[2 * q + 1] += __uint_as_float(w4[q] & 0xffff0000u);
      }
    }
    uint32_t o4[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const __nv_bfloat162 hh = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      o4[q] = *reinterpret_cast<const uint32_t*>(&hh);
    }
    *reinterpret_cast<uint4*>(out + (long long)t * h + c * 8) = make_uint4(o4[0], o4[1], o4[2], o4[3]);
  }
}

}  // namespace b200

// ids int32 [m, k] (global ids, negative = empty slot) -> counts int32 [world], offsets int32 [world + 1], pos int32
// [m, world], send_tok int32 [m * min(world, k)] (device buffers). 0 <= m <= 8192 * 8, world <= 16.
extern "C" int b200moe_ep_plan(const int* ids, int m, int k, int world, int experts_per_rank, int* counts, int* offsets, int* pos,
                               int* send_tok, void* stream) {
  if (!counts || !offsets || (m > 0 && (!ids || !pos || !send_tok))) return B200MOE_ERR_ARG;
  if (m < 0 || k < 1 || world < 1 || world > kEpMaxWorld || experts_per_rank < 1) return B200MOE_ERR_SHAPE;
  if (m == 0) {   // a rank with an empty batch still takes part in the exchange: it sends nothing to anybody
    B200_CUDA_TRY(cudaMemsetAsync(counts, 0, sizeof(int) * world, (cudaStream_t)stream));
    B200_CUDA_TRY(cudaMemsetAsync(offsets, 0, sizeof(int) * (world + 1), (cudaStream_t)stream));
    return B200MOE_OK;
  }
  k_ep_plan<<<1, 1024, 0, (cudaStream_t)stream>>>(ids, m, k, world, experts_per_rank, counts, offsets, pos, send_tok);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// rows [0, offsets[world]) of sx bf16 [rows, h] and meta int32 [rows, 2k] (local ids, then the weights' float bits)
extern "C" int b200moe_ep_gather(const void* x, const int* ids, const float* wts, const int* send_tok, const int* offsets, int h, int k, int world,
                                 int experts_per_rank, int max_rows, void* sx, int* meta, void* stream) {
  if (h <= 0 || h % 8 || k < 1 || world < 1 || world > kEpMaxWorld || max_rows < 0) return B200MOE_ERR_SHAPE;
  if (max_rows == 0) return B200MOE_OK;   // nothing to send (an empty batch): the buffers may be null
  if (!x || !ids || !wts || !send_tok || !offsets || !sx || !meta) return B200MOE_ERR_ARG;
  const int grid = max_rows < 148 * 16 ? max_rows : 148 * 16;
  k_ep_gather<<<grid, 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ids, wts, send_tok, offsets, h, k, world, experts_per_rank,
                                                      (__nv_bfloat16*)sx, meta);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// back bf16 [rows, h] (the partial rows in send-buffer order), pos int32 [m, world] -> out bf16 [m, h]
extern "C" int b200moe_ep_combine_rows(const void* back, const int* pos, int m, int h, int world, void* out, void* stream) {
  if (m > 0 && (!back || !pos || !out)) return B200MOE_ERR_ARG;
  if (m < 0 || h <= 0 || h % 8 || world < 1 || world > kEpMaxWorld) return B200MOE_ERR_SHAPE;
  if (m == 0) return B200MOE_OK;
  const int total = m * (h / 8);
  int grid = (total + 255) / 256;
  if (grid > 148 * 16) grid = 148 * 16;
  k_ep_combine_rows<<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)back, pos, m, h, world, (__nv_bfloat16*)out);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// ---------------------------------------------------------------------------------------------------------------------
// Flagged-word form of the peer-store exchange (see k_ep_dispatch_ll). peers_in: host array of `world` device pointers, entry
// d = where this rank's block starts inside rank d's flagged receive area (uint2 [cap][h/2 + 2k] per source rank); in: this
// rank's own receive area (uint2 [world][cap][h/2 + 2k]); rx / rid / rw: the plain arrays the layer call takes;
// calls: device uint32 [2], zeroed once together with the areas; status: device int32, 0 or 1 + the rank whose words never
// arrived. One layer call = b200moe_ep_dispatch_ll, the local layer, b200moe_ep_return_combine_ll, in that order.
extern "C" int b200moe_ep_dispatch_ll(const void* x, const int* ids, const float* wts, int m, int h, int k, int world, int experts_per_rank,
                                      int cap, void* const* peers_in, const void* in, void* rx, int* rid, float* rw, unsigned* calls, int* status,
                                      void* stream) {
  if ((m > 0 && (!x || !ids || !wts)) || !peers_in || !in || !rx || !rid || !rw || !calls || !status) return B200MOE_ERR_ARG;
  if (m < 0 || m > cap || h <= 0 || h % 8 || k < 1 || 2 * k > 128 || world < 1 || world > kEpMaxWorld || experts_per_rank < 1 || cap < 1)
    return B200MOE_ERR_SHAPE;
  if ((long long)cap * world > kEpMaxWaitingBlocks) return B200MOE_ERR_LIMIT;
  EpLLPeers D;
  for (int d = 0; d < kEpMaxWorld; ++d) {
    D.p[d] = d < world ? (uint2*)peers_in[d] : nullptr;
    if (d < world && (!D.p[d] || ((uintptr_t)D.p[d] & 7))) return B200MOE_ERR_ARG;
  }
  k_ep_dispatch_ll<<<dim3(cap, world), 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, ids, wts, m, h, k, experts_per_rank, cap, D,
                                                                        (const uint2*)in, (__nv_bfloat16*)rx, rid, rw, calls, status);
  B200_LAUNCH_CHECK();
  return B200MOE_OK;
}

// yl bf16 [world * cap, h]: this rank's partial rows (block s for source s); rid: the ids b200moe_ep_dispatch_ll received
// (which rows carry anything); peers_back: host array, entry s = where block `rank` starts inside rank s's flagged return
// area (uint2 [cap][h/2] per computing rank); back: this rank's own return area (uint2 [world][cap][h/2], then `world` marker
// words: (world * cap * h/2 + world) * 8 bytes); ids: the caller's
// global top-k ids of this call (int32 [m, k]); out bf16 [m, h].
extern "C" int b200moe_ep_return_combine_ll(const void* yl, const int* rid, int world, int cap, int h, int k, int rank, int experts_per_rank,
                                            void* const* peers_back, const void* back, const int* ids, int m, void* out, unsigned* calls,
                                            int* status, void* stream) {
  if (!yl || !rid || !peers_back || !back || !calls || !status || (m > 0 && (!ids || !out))) return B200MOE_ERR_ARG;
  if (world < 1 || world > kEpMaxWorld || cap < 1 || h <= 0 || h % 8 || k < 1 || rank < 0 || rank >= world || m < 0 || m > cap ||
      experts_per_rank < 1)
    return B200MOE_ERR_SHAPE;
  if ((long long)cap * world > kEpMaxWaitingBlocks) return B200MOE_ERR_LIMIT;
  EpLLPeers B;
  for (int d = 0; d < kEpMaxWorld; ++d) {
    B.p[d] = d < world ? (uint2*)peers_back[d] : nullptr;
    if (d < world && (!B.p[d] || ((uintptr_t)B.p[d] & 7))) return B200MOE_ERR_ARG;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(cap, world), cfg.blockDim = dim3(128), cfg.dynamicSmemBytes = 0, cfg.stream = (cudaStream_t)stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr, cfg.numAttrs = 1;
  B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, k_ep_return_ll, (const __nv_bfloat16*)yl, rid, cap, h, k, rank, world, experts_per_rank, B,
                                   (const uint2*)back, ids, m, (__nv_bfloat16*)out, calls, status));
  return B200MOE_OK;
}
