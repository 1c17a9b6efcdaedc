// Token-to-expert routing: counts, exclusive scan, stable permutation. Bit-exact with the torch router of
// sm120fp4/kernels/fc1_w4a16.py:272-279 (stable argsort of the flattened ids) and with the fixed-size padded form the
// reference's GPU router writes (sm120fp4/kernels/moe_w4a16.py:48-83: unused expert slots -1, unused offsets P).
// The reference ranks each pair with an O(P^2) loop in one block; here a stable counting sort over chunks of pairs
// scales to prefill sizes (P = 65,536 and beyond): no atomic decides any position.
#include "common.cuh"
#include <atomic>

namespace b200 {

constexpr int ROUTE_MAXE = 1024;   // experts per layer the router takes
constexpr int ROUTE_CHUNK = 512;   // pairs per chunk (one warp walks a chunk in order)

// Pass 1: per-chunk histogram. One block of 128 threads per chunk; counts are order-independent.
__global__ void __launch_bounds__(128) k_route_hist(const int* __restrict__ ids, int P, int E, int* __restrict__ hist,
                                                    int* __restrict__ bad) {
  extern __shared__ int sh[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  const int p0 = blockIdx.x * ROUTE_CHUNK, p1 = min(P, p0 + ROUTE_CHUNK);
  for (int p = p0 + threadIdx.x; p < p1; p += blockDim.x) {
    const int e = ids[p];
    if (e < 0) continue;                 // empty slot
    if (e >= E) { *bad = 1; continue; }
    atomicAdd(&sh[e], 1);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[(long long)blockIdx.x * E + e] = sh[e];
}

// Pass 2 (one block of 1024 threads): per expert, exclusive scan of the chunk counts in place (chunk-local base of
// that expert); then scan over experts for the expert bases and the touched-expert index; write the tables.
__global__ void __launch_bounds__(1024) k_route_scan(int* __restrict__ hist, int nchunks, int P, int E, int Umax,
                                                     int* __restrict__ experts, int* __restrict__ offsets,
                                                     int* __restrict__ expert_base /* [E], start of expert e in pairs */,
                                                     int* __restrict__ num_touched) {
  __shared__ int base[ROUTE_MAXE], uidx[ROUTE_MAXE];
  const int t = threadIdx.x;
  int c = 0;
  if (t < E) {
    for (int b0 = 0; b0 < nchunks; b0 += 8) {   // eight independent loads in flight, then their running sums
      int v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = b0 + i < nchunks ? hist[(long long)(b0 + i) * E + t] : 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (b0 + i < nchunks) hist[(long long)(b0 + i) * E + t] = c;
        c += v[i];
      }
    }
  }
  base[t] = c;
  uidx[t] = c > 0 ? 1 : 0;
  __syncthreads();
  for (int o = 1; o < ROUTE_MAXE; o <<= 1) {   // inclusive Hillis-Steele scans of counts and touched flags
    const int b = t >= o ? base[t - o] : 0, u = t >= o ? uidx[t - o] : 0;
    __syncthreads();
    base[t] += b;
    uidx[t] += u;
    __syncthreads();
  }
  const int U = uidx[ROUTE_MAXE - 1];
  const int routed = base[ROUTE_MAXE - 1];   // pairs with a non-negative id (= P when no slot is empty)
  if (t < E) {
    expert_base[t] = base[t] - c;
    if (c > 0 && uidx[t] - 1 < Umax) {
      experts[uidx[t] - 1] = t;
      offsets[uidx[t] - 1] = base[t] - c;
    }
  }
  for (int u = U + t; u < Umax; u += blockDim.x) {
    experts[u] = -1;
    offsets[u + 1] = routed;
  }
  if (t == 0) {
    if (U <= Umax) offsets[U] = routed;
    if (num_touched) *num_touched = U;
  }
}

// Pass 3: one warp per chunk walks its pairs in index order, 32 at a time. Within a step, pairs of the same expert are
// ranked by lane; across steps a per-expert running count in shared memory carries the order. Position of pair p =
// expert_base[e] + (pairs of e in earlier chunks) + (pairs of e earlier in this chunk).
__global__ void __launch_bounds__(32) k_route_place(const int* __restrict__ ids, int P, int E, const int* __restrict__ hist,
                                                    const int* __restrict__ expert_base, int* __restrict__ pairs) {
  extern __shared__ int run[];
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) run[e] = expert_base[e] + hist[(long long)blockIdx.x * E + e];
  __syncwarp();
  const int p0 = blockIdx.x * ROUTE_CHUNK, p1 = min(P, p0 + ROUTE_CHUNK);
  int mine[ROUTE_CHUNK / 32];   // this lane's ids of the chunk, all loads in flight at once
#pragma unroll
  for (int k = 0; k < ROUTE_CHUNK / 32; ++k) mine[k] = p0 + 32 * k + lane < p1 ? ids[p0 + 32 * k + lane] : -1;
#pragma unroll
  for (int k = 0; k < ROUTE_CHUNK / 32; ++k) {
    const int s = p0 + 32 * k;
    if (s >= p1) break;
    const int p = s + lane;
    int e = mine[k];
    if (e < 0 || e >= E) e = -1;
    const unsigned active = __ballot_sync(0xffffffffu, e >= 0);
    if (e >= 0) {
      const unsigned peers = __match_any_sync(active, e);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      const int pos = run[e] + rank;
      pairs[pos] = p;
      __syncwarp(active);
      if (rank == __popc(peers) - 1) run[e] += __popc(peers);   // the last peer advances the running count
    }
    __syncwarp();
  }
}

// The whole router in one launch for small batches (P <= kRouteSmallMaxP pairs, E <= 256 experts: decode-sized and mid-sized
// batches, where three launches cost more than the work). One block of 32 warps; warp w owns the contiguous pairs
// [w * L, (w + 1) * L). Counts per (warp, expert) in shared memory, a scan over the warps per expert and over the experts,
// then every warp walks its pairs in index order exactly as k_route_place does. Same tables, bit for bit.
constexpr int kRouteSmallMaxP = 4096, kRouteSmallMaxE = 256;

__global__ void __launch_bounds__(1024) k_route_small(const int* __restrict__ ids, int P, int E, int Umax, int* __restrict__ experts,
                                                      int* __restrict__ offsets, int* __restrict__ pairs, int* __restrict__ bad,
                                                      int* __restrict__ num_touched) {
  __shared__ int wc[32][kRouteSmallMaxE];     // pairs of expert e in warp w's range, then the start of that range's run in `pairs`
  __shared__ int tot[kRouteSmallMaxE], uidx[kRouteSmallMaxE];
  __shared__ int s_bad;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < 32 * kRouteSmallMaxE; i += 1024) (&wc[0][0])[i] = 0;
  if (tid == 0) s_bad = 0;
  __syncthreads();
  const int L = ((P + 31) / 32 + 31) & ~31;   // pairs per warp, a multiple of 32
  const int p0 = warp * L, p1 = min(P, p0 + L);
  for (int p = p0 + lane; p < p1; p += 32) {
    const int e = ids[p];
    if (e < 0) continue;
    if (e >= E) { s_bad = 1; continue; }
    atomicAdd(&wc[warp][e], 1);
  }
  __syncthreads();
  if (tid < kRouteSmallMaxE) {   // thread e: exclusive scan of expert e's counts over the warps
    int c = 0;
    for (int w = 0; w < 32; ++w) { const int v = wc[w][tid]; wc[w][tid] = c; c += v; }
    tot[tid] = c;
  }
  __syncthreads();
  if (warp == 0) {               // scan over the experts: bases and touched-expert indices (8 experts per lane)
    int c[8], sc = 0, sf = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) { c[i] = tot[lane * 8 + i]; sc += c[i]; sf += c[i] > 0; }
    int ic = sc, iff = sf;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, ic, o), b = __shfl_up_sync(0xffffffffu, iff, o);
      if (lane >= o) { ic += a; iff += b; }
    }
    int rc = ic - sc, rf = iff - sf;
    const int routed = __shfl_sync(0xffffffffu, ic, 31), U = __shfl_sync(0xffffffffu, iff, 31);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane * 8 + i;
      tot[e] = rc;                          // start of expert e in `pairs`
      if (c[i] > 0) {
        if (rf < Umax) { experts[rf] = e; offsets[rf] = rc; }
        ++rf;
      }
      uidx[e] = rf;
      rc += c[i];
    }
    for (int u = U + lane; u < Umax; u += 32) { experts[u] = -1; offsets[u + 1] = routed; }
    if (lane == 0) {
      if (U <= Umax) offsets[U] = routed;
      if (num_touched) *num_touched = U;
      if (bad) *bad = s_bad;
    }
  }
  __syncthreads();
  for (int e = lane; e < kRouteSmallMaxE; e += 32) wc[warp][e] += tot[e];   // this warp's running position per expert
  __syncwarp();
  for (int s = p0; s < p1; s += 32) {
    const int p = s + lane;
    int e = p < p1 ? ids[p] : -1;
    if (e < 0 || e >= E) e = -1;
    const unsigned active = __ballot_sync(0xffffffffu, e >= 0);
    if (e >= 0) {
      const unsigned peers = __match_any_sync(active, e);
      const int rank = __popc(peers & ((1u << lane) - 1u));
      pairs[wc[warp][e] + rank] = p;
      __syncwarp(active);
      if (rank == __popc(peers) - 1) wc[warp][e] += __popc(peers);
    }
    __syncwarp();
  }
}

}  // namespace b200

using namespace b200;

extern "C" long long b200moe_route_workspace_bytes(int P, int E) {
  if (P < 0 || E <= 0) return B200MOE_ERR_ARG;
  const long long nchunks = (P + ROUTE_CHUNK - 1) / ROUTE_CHUNK;
  return (nchunks * E + E + 2) * (long long)sizeof(int);
}

// ids int32 [P] -> experts int32 [Umax], offsets int32 [Umax+1], pairs int32 [P]; Umax slots as the caller sized them
// (the reference uses min(E, P)). workspace: b200moe_route_workspace_bytes(P, E) bytes of device memory.
extern "C" int b200moe_route(const int* ids, int P, int E, int Umax, int* experts, int* offsets, int* pairs, void* workspace,
                             long long workspace_bytes, void* stream) {
  if (!offsets || !workspace || P < 0 || Umax < 0) return B200MOE_ERR_ARG;
  if ((P > 0 && (!ids || !pairs)) || (Umax > 0 && !experts)) return B200MOE_ERR_ARG;
  if (E <= 0 || E > ROUTE_MAXE) return B200MOE_ERR_SHAPE;
  if (workspace_bytes < b200moe_route_workspace_bytes(P, E)) return B200MOE_ERR_WORKSPACE;
  cudaStream_t st = (cudaStream_t)stream;
  const int nchunks = (P + ROUTE_CHUNK - 1) / ROUTE_CHUNK;
  int* hist = (int*)workspace;
  int* expert_base = hist + (long long)nchunks * E;
  int* bad = expert_base + E;
  int* num_touched = bad + 1;
  if (P > 0 && P <= kRouteSmallMaxP && E <= kRouteSmallMaxE) {   // small batch: one launch
    k_route_small<<<1, 1024, 0, st>>>(ids, P, E, Umax, experts, offsets, pairs, bad, num_touched);
    B200_LAUNCH_CHECK();
    return B200MOE_OK;
  }
  B200_CUDA_TRY(cudaMemsetAsync(bad, 0, 2 * sizeof(int), st));
  if (nchunks > 0) {
    k_route_hist<<<nchunks, 128, E * sizeof(int), st>>>(ids, P, E, hist, bad);
    B200_LAUNCH_CHECK();
  }
  k_route_scan<<<1, 1024, 0, st>>>(hist, nchunks, P, E, Umax, experts, offsets, expert_base, num_touched);
  B200_LAUNCH_CHECK();
  if (nchunks > 0) {
    k_route_place<<<nchunks, 32, E * sizeof(int), st>>>(ids, P, E, hist, expert_base, pairs);
    B200_LAUNCH_CHECK();
  }
  return B200MOE_OK;
}

// An expert id >= E is skipped by the kernels (its pair appears in no table, the tables of the other pairs are as if its
// slot were empty) and raises a flag inside the scratch memory. This reads the flag of the last call that used `workspace`
// with the same P and E: 0, or B200MOE_ERR_ARG. Synchronises the stream.
static int route_read_bad(const int* scratch, int P, int E, cudaStream_t st) {
  const long long nchunks = (P + ROUTE_CHUNK - 1) / ROUTE_CHUNK;
  int bad = 0;
  B200_CUDA_TRY(cudaMemcpyAsync(&bad, scratch + nchunks * E + E, sizeof(int), cudaMemcpyDeviceToHost, st));
  B200_CUDA_TRY(cudaStreamSynchronize(st));
  return bad ? B200MOE_ERR_ARG : B200MOE_OK;
}

extern "C" int b200moe_route_status(const void* workspace, int P, int E, void* stream) {
  if (!workspace || P < 0 || E <= 0 || E > ROUTE_MAXE) return B200MOE_ERR_ARG;
  return route_read_bad((const int*)workspace, P, E, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------------------------------
// Router for callers that cannot hand over scratch memory.
//
// Some hosts of this library own no allocator: an inference server that has finished its memory-profiling pass and
// forbids any further device allocation, or a plugin that is only ever given its input and output buffers. For them the
// chunk histograms and expert bases of the router live in a fixed device array inside the library image instead of a
// caller-provided workspace. Every GPU that loads the library carries these kRouteStaticInts * 4 bytes (about 129 KiB)
// until the process exits.
constexpr int kRouteStaticMaxPairs = 65536;   // 8192 tokens x top-8
constexpr int kRouteStaticMaxExperts = 256;
constexpr int kRouteStaticInts = (kRouteStaticMaxPairs / b200::ROUTE_CHUNK) * kRouteStaticMaxExperts + kRouteStaticMaxExperts + 2;
static __device__ __align__(256) int g_route_static[kRouteStaticInts];

// In host code `g_route_static` is only a handle for the symbol, not an address a kernel can use: the device address is
// looked up per device with cudaGetSymbolAddress, with that device current, the first time the entry point runs there.
static int route_static_address(int** out) {
  constexpr int kMaxDevices = 64;
  static std::atomic<int*> addr[kMaxDevices];   // zero-initialised; threads that race on a first call store the same value
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return B200MOE_ERR_DEVICE;
  int* p = addr[dev].load(std::memory_order_acquire);
  if (!p) {
    B200_CUDA_TRY(cudaGetSymbolAddress((void**)&p, g_route_static));
    addr[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return B200MOE_OK;
}

// Same tables as b200moe_route, with no workspace argument and no allocation of any kind inside the call.
//  * limits: P <= 65536 pairs and E <= 256 experts, otherwise B200MOE_ERR_LIMIT.
//  * the first call on a device resolves the address of the built-in scratch (a synchronous runtime query), so make that
//    first call before starting a stream capture on that device.
//  * all calls on a device share the one scratch array: two calls whose kernels may overlap on the GPU (different streams)
//    race on it. The array keeps what the previous call left; the cells that must start from zero (the bad-id flag and the
//    touched-expert count) are cleared on the stream at the start of every call, the rest is fully rewritten.
extern "C" int b200moe_route_static(const int* ids, int P, int E, int Umax, int* experts, int* offsets, int* pairs, void* stream) {
  if (!offsets || P < 0 || Umax < 0) return B200MOE_ERR_ARG;
  if ((P > 0 && (!ids || !pairs)) || (Umax > 0 && !experts)) return B200MOE_ERR_ARG;
  if (E <= 0) return B200MOE_ERR_SHAPE;
  if (P > kRouteStaticMaxPairs || E > kRouteStaticMaxExperts) return B200MOE_ERR_LIMIT;
  int* scratch = nullptr;
  const int rc = route_static_address(&scratch);
  if (rc != B200MOE_OK) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const int nchunks = (P + ROUTE_CHUNK - 1) / ROUTE_CHUNK;
  int* hist = scratch;
  int* expert_base = hist + (long long)nchunks * E;
  int* bad = expert_base + E;
  int* num_touched = bad + 1;
  B200_CUDA_TRY(cudaMemsetAsync(bad, 0, 2 * sizeof(int), st));
  if (nchunks > 0) {
    k_route_hist<<<nchunks, 128, E * sizeof(int), st>>>(ids, P, E, hist, bad);
    B200_LAUNCH_CHECK();
  }
  k_route_scan<<<1, 1024, 0, st>>>(hist, nchunks, P, E, Umax, experts, offsets, expert_base, num_touched);
  B200_LAUNCH_CHECK();
  if (nchunks > 0) {
    k_route_place<<<nchunks, 32, E * sizeof(int), st>>>(ids, P, E, hist, expert_base, pairs);
    B200_LAUNCH_CHECK();
  }
  return B200MOE_OK;
}

// The bad-id flag of the last b200moe_route_static call on the current device (same P and E): 0 or B200MOE_ERR_ARG.
// Synchronises the stream; allocates nothing.
extern "C" int b200moe_route_static_status(int P, int E, void* stream) {
  if (P < 0 || E <= 0) return B200MOE_ERR_ARG;
  if (P > kRouteStaticMaxPairs || E > kRouteStaticMaxExperts) return B200MOE_ERR_LIMIT;
  int* scratch = nullptr;
  const int rc = route_static_address(&scratch);
  if (rc != B200MOE_OK) return rc;
  return route_read_bad(scratch, P, E, (cudaStream_t)stream);
}
