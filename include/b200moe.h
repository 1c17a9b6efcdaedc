/* b200moe: C ABI of the B200-native (sm_100a) NVFP4 fused-MoE library.
 *
 * Plain pointers and sizes only: no torch types, no exceptions, no device allocation inside any call. Every device
 * buffer belongs to the caller; `stream` is a cudaStream_t passed as void*. All functions return 0 on success or a
 * negative B200MOE_ERR_* code; kernels are enqueued on `stream` and nothing synchronises unless stated.
 *
 * Each entry point names the interface of the reference project (sm120fp4) that it replaces, by file:line.
 */
#ifndef B200MOE_H
#define B200MOE_H

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_OK 0
#define B200MOE_ERR_ARG (-1)       /* null pointer, negative size, misaligned buffer, expert id out of range */
#define B200MOE_ERR_SHAPE (-2)     /* a dimension the kernels do not take */
#define B200MOE_ERR_CUDA (-3)      /* a CUDA call failed: b200moe_last_cuda_error() */
#define B200MOE_ERR_DEVICE (-4)    /* not an sm_100 device / tensor-map driver entry point missing */
#define B200MOE_ERR_TIMEOUT (-5)   /* a bounded device-side wait ran out */
#define B200MOE_ERR_WORKSPACE (-6) /* workspace too small */
#define B200MOE_ERR_LIMIT (-7)     /* size beyond a stated maximum */
#define B200MOE_ERR_RANGE (-8)     /* an FC1 activation exceeded the range of the activation scale and was clipped */
#define B200MOE_ERR_ORDER (-9)     /* topk_ids / topk_weights changed while the call was running */

typedef struct b200moe_layer b200moe_layer; /* opaque decode-layer handle (host memory) */

int b200moe_version(void);
const char* b200moe_error_string(int code);
const char* b200moe_last_cuda_error(void);

/* ---- block-scale layout: sm120fp4/layouts.py:56-68 (to_128x4) and :71-78 (from_128x4), batched over `batch`
 * matrices. sf_linear u8 [batch, rows, cols]; sf_swizzled u8 [batch, pad128(rows) * pad4(cols)], padding written 0. */
int b200moe_to_128x4(const void* sf_linear, void* sf_swizzled, int batch, int rows, int cols, void* stream);
int b200moe_from_128x4(const void* sf_swizzled, void* sf_linear, int batch, int rows, int cols, void* stream);

/* ---- quantizer: sm120fp4/reference.py:68-71 (global_scale_for) and :74-90 (quantize_nvfp4). dtype 0 = bf16, 1 = f32.
 * b200moe_global_scale: gs_out[0] = 2688 / max(amax|x|, 1e-12) with the reference's rounding; amax_scratch_u32 is 4
 * bytes of device scratch. b200moe_quantize_nvfp4: global_scale holds one value (gs_rows 0) or one per gs_rows
 * destination rows (stacked experts); destination row r quantises source row src_row[r] (null: r; negative:
 * zero codes and scales); packed u8 [rows, K/2]; sf u8 row-major [rows, K/16] (sf_layout 0) or 128x4-swizzled over
 * [rows, K/16] (sf_layout 1; the caller sizes the buffer for the padded extent). Bit-exact with the reference. */
int b200moe_global_scale(const void* x, int dtype, long long n, void* amax_scratch_u32, float* gs_out, void* stream);
int b200moe_global_scale_grouped(const void* x, int dtype, int groups, long long group_elems, void* amax_scratch_u32,
                                 float* gs_out, void* stream); /* one scale per group (per expert); scratch 4*groups bytes */
int b200moe_quantize_nvfp4(const void* x, int dtype, const int* src_row, int rows, int K, const float* global_scale,
                           int gs_rows, void* packed, void* sf, int sf_layout, void* stream);

/* ---- router: sm120fp4/kernels/moe_w4a16.py:85-91 (route; padded form of k_route :48-83) and the torch router of
 * sm120fp4/kernels/fc1_w4a16.py:272-279. ids i32 [P] -> experts i32 [Umax] (ascending, -1 padding), offsets i32
 * [Umax+1] (exclusive scan, P padding), pairs i32 [P] (pair indices grouped by expert, ascending within). */
long long b200moe_route_workspace_bytes(int P, int E);
int b200moe_route(const int* ids, int P, int E, int Umax, int* experts, int* offsets, int* pairs, void* workspace,
                  long long workspace_bytes, void* stream);
/* An id >= E is skipped (its pair appears in no table) and raises a flag in the workspace; this reads the flag of the last
 * call that used `workspace` with the same P and E: 0 or B200MOE_ERR_ARG (the reference's router has no such check: its
 * ids come straight from top-k, sm120fp4/kernels/moe_w4a16.py:48-83). Synchronises the stream. */
int b200moe_route_status(const void* workspace, int P, int E, void* stream);

/* Router for hosts that cannot provide scratch memory (no counterpart in the reference). Identical tables to b200moe_route,
 * but the intermediate histograms sit in a fixed array inside the library (about 129 KiB per GPU that loads it), so the call
 * allocates nothing and takes no workspace. Meant for callers with no allocator of their own: a server that froze its
 * memory budget after start-up, a plugin that only receives its input and output buffers. Limits: P <= 65536, E <= 256
 * (B200MOE_ERR_LIMIT beyond). The first call on each device looks up the array's device address - issue it before any
 * stream capture. Calls on one device share the array: do not let two of them overlap on the GPU. */
int b200moe_route_static(const int* ids, int P, int E, int Umax, int* experts, int* offsets, int* pairs, void* stream);
/* bad-id flag of the last b200moe_route_static call on the current device (same P, E); synchronises, allocates nothing */
int b200moe_route_static_status(int P, int E, void* stream);

/* ---- decode layer (M <= 16 tokens, W4A16): sm120fp4/vllm_backend.py:95-121 (Weights) and :147-190 (forward/_slice).
 * q1 u8 [E, 2I, H/2] rows [up ; gate]; s1 u8 [E, pad128(2I) * pad4(H/16)] 128x4-swizzled per expert; q2 u8 [E, H, I/2];
 * s2 u8 [E, pad128(H) * pad4(I/16)] 128x4-swizzled per expert; alpha f32 [E] (weight_scale_2). H % 128 == 0,
 * I % 64 == 0, E <= 256, top_k <= 16. The handle keeps the pointers; the buffers must outlive it. */
int b200moe_layer_create(b200moe_layer** out, int E, int H, int I, int top_k, const void* q1, const void* s1_128x4,
                         const float* alpha1, const void* q2, const void* s2_128x4, const float* alpha2);
void b200moe_layer_destroy(b200moe_layer* layer);
long long b200moe_layer_workspace_bytes(const b200moe_layer* layer);
int b200moe_layer_workspace_init(const b200moe_layer* layer, void* workspace, long long workspace_bytes, void* stream);
int b200moe_layer_sm_count(const b200moe_layer* layer);
/* tcgen05 decode path: the kernel-native weight copy - every (expert, block, K box) tile as one contiguous 18 KB record of
 * codes (shared-memory image) + scale tiles - built once per layer into caller-owned device memory of about the size of
 * the weights (the counterpart of the load-time re-layout in sm120fp4/vllm_backend.py:193-206; the caller may drop the
 * checkpoint-layout codes afterwards if it only decodes). After prepack, b200moe_decode_forward runs the tcgen05 kernel;
 * b200moe_layer_set_decode_impl picks 0 = automatic, 1 = mma.sync kernel, 2 = tcgen05 kernel; b200moe_layer_set_act_scale
 * sets the global scale of the first NVFP4 term of the FC1->FC2 activations (default 8). */
long long b200moe_layer_prepack_bytes(const b200moe_layer* layer);
int b200moe_layer_prepack(b200moe_layer* layer, void* buffer, long long buffer_bytes, void* stream);
int b200moe_layer_set_decode_impl(b200moe_layer* layer, int impl);
/* Forget the checkpoint-layout codes and scales (the caller may free them): from then on only the tcgen05 paths run; the
 * mma.sync kernel and b200moe_decode_fc1 / _fc2 return B200MOE_ERR_ARG. Needs b200moe_layer_prepack. The reference keeps a
 * single copy of the weights too: its load-time re-layout is in place (sm120fp4/vllm_backend.py:193-206). */
int b200moe_layer_release_checkpoint(b200moe_layer* layer);
int b200moe_layer_set_act_scale(b200moe_layer* layer, float first_term_global_scale);

/* ---- W4A4 prefill for any M <= max_tokens: the layer's own tcgen05 kind::mxf4nvf4 grouped GEMM in place of the reference's
 * hand-off to FlashInfer's CUTLASS MoE (sm120fp4/vllm_backend.py:123-145 enable_cutlass_prefill, :161-168 the call); the
 * arithmetic is the reference's W4A4 oracle (sm120fp4/kernels/bench_moe_baseline.py:53-74, act_quant=True). Needs
 * b200moe_layer_prepack. gs_x, gs_a: global scales of the two activation quantisations (1 / input scales). */
long long b200moe_prefill_workspace_bytes(const b200moe_layer* layer, int max_tokens);
int b200moe_prefill_forward(const b200moe_layer* layer, const void* x_bf16, const int* topk_ids, const float* topk_weights, int M,
                            void* out_bf16, void* workspace, long long workspace_bytes, int max_tokens, float gs_x, float gs_a,
                            void* stream);
int b200moe_prefill_status(const b200moe_layer* layer, const void* workspace, int max_tokens, void* stream);
/* Byte offsets inside a prefill workspace sized for max_tokens, so that a tool or a test can read back what each stage of the
 * last call wrote (the reference exposes its intermediates the same way, as tensors: sm120fp4/kernels/bench_moe_baseline.py:
 * 53-74 returns them from `reference`). out14 = experts, offsets, pairs (router tables), ntiles, tile_expert, tile_first,
 * tile_end (128-row tiles: expert, first and end index into pairs), row_pair [tiles*128], dst_row [pairs], x records,
 * activation records, weighted bf16 rows, tile capacity, total bytes. A record is 18,432 bytes per (tile, 256-value K box):
 * row r, 16-value block b at r*128 + (((b>>1) ^ (r&7)) << 4) + (b&1)*8 (8 code bytes), its scale byte at 16384 + (b>>2)*512 +
 * (r&31)*16 + (r>>5)*4 + (b&3) - i.e. four 128x4 scale tiles. */
int b200moe_prefill_workspace_map(const b200moe_layer* layer, int max_tokens, long long* out14);

/* forward: x bf16 [M, H], topk_ids i32 [M, top_k], topk_weights f32 [M, top_k] -> out bf16 [M, H]; one launch
 * (routing + FC1 + SiLU*mul + FC2 + weighted combine). Replaces Weights._slice, sm120fp4/vllm_backend.py:174-190. */
int b200moe_decode_forward(const b200moe_layer* layer, const void* x_bf16, const int* topk_ids, const float* topk_weights,
                           int M, void* out_bf16, void* workspace, long long workspace_bytes, void* stream);
/* The same with flags. B200MOE_ORDERED: the two kernels of the call are ordinary stream-ordered launches. By default they are
 * launched programmatically, so that the call's prologue and weight stream overlap the tail of whatever precedes it in
 * the stream, and topk_ids / topk_weights are read at kernel entry: they must be complete when the kernel BEFORE this call
 * starts (true for any producer that does not itself release its successors early, or that releases them only after these
 * tensors are written and fenced, as b200moe_ep_dispatch_ll does). A violation is detected (the inputs are
 * re-read after the stream dependency has resolved) and reported by b200moe_layer_status as B200MOE_ERR_ORDER. This is the
 * per-call form of the reference's module-wide switches fc1_set_pdl / fc2_set_pdl (sm120fp4/vllm_backend.py:174-190). */
#define B200MOE_ORDERED 1
int b200moe_decode_forward_ex(const b200moe_layer* layer, const void* x_bf16, const int* topk_ids, const float* topk_weights,
                              int M, void* out_bf16, void* workspace, long long workspace_bytes, int flags, void* stream);
/* b200moe_decode_forward for a caller whose tensors live in host memory: x bf16 [M, H], ids int32 [M, top_k], weights f32
 * [M, top_k] in, out bf16 [M, H] back. The inputs go through staging buffers inside the workspace (three small copies on
 * `stream`); a page-locked output buffer is written by the kernel directly across the host link, a pageable one is copied
 * back. Everything is enqueued on `stream`, nothing synchronises. M <= 16. Replaces the same call
 * site as b200moe_decode_forward (sm120fp4/vllm_backend.py:174-190) for hosts that do not hold device tensors. */
int b200moe_decode_forward_host(const b200moe_layer* layer, const void* x_host, const int* ids_host, const float* wts_host, int M,
                                void* out_host, void* workspace, long long workspace_bytes, void* stream);

/* FC1 alone -> act bf16 [M*top_k, I], row = pair index: sm120fp4/kernels/fc1_w4a16.py:251-262, fc1_mma.py:266-282. */
int b200moe_decode_fc1(const b200moe_layer* layer, const void* x_bf16, const int* topk_ids, const float* topk_weights, int M,
                       void* act_bf16, void* workspace, long long workspace_bytes, void* stream);
/* FC2 alone from act bf16 [M*top_k, I]: sm120fp4/kernels/fc2_w4a16.py:276-279, fc2_mma_pf.py:403-421. */
int b200moe_decode_fc2(const b200moe_layer* layer, const void* act_bf16, const int* topk_ids, const float* topk_weights, int M,
                       void* out_bf16, void* workspace, long long workspace_bytes, void* stream);
/* routing tables written by the last decode call, in the router's padded form (device-to-device copies on stream) */
int b200moe_layer_route_tables(const b200moe_layer* layer, const void* workspace, int M, int* experts, int* offsets,
                               int* pairs, void* stream);
/* Byte offsets inside a decode workspace of what the tcgen05 decode kernel computed with in the last call, for tools and tests
 * (as b200moe_prefill_workspace_map): out8 = the x operand (per 256-value K box N rows of 128 code bytes in the 128-byte
 * swizzle - row 4*token + term, 16-byte chunk c at c ^ (row & 7) - then ceil(H/64) scale tiles of 512 bytes), its 1/g_t per
 * row (float [N]), the activation slabs ([touched expert][K box of I]: N rows of 128 code bytes + four 512-byte scale tiles),
 * slab bytes for N = 16, 32, 64 (tokens <= 4, 8, 16), the activation scale (float bits), slab capacity in experts. */
int b200moe_layer_workspace_map(const b200moe_layer* layer, long long* out8);
/* status words of the workspace; synchronises the stream. 0, B200MOE_ERR_TIMEOUT, B200MOE_ERR_ARG (bad expert id),
 * B200MOE_ERR_ORDER (routing inputs changed under the call) or B200MOE_ERR_RANGE (an FC1 activation above 2688 / act scale
 * was clipped; the last two are cleared by the read) */
int b200moe_layer_status(const b200moe_layer* layer, const void* workspace, void* stream);

/* single-tile check of the tcgen05 building blocks (TMEM, descriptors, scale copies, kind::mxf4nvf4 MMA): d f32 [128, N]
 * = dequant(a)[128, K] x dequant(b)[N, K]^T with 128x4-swizzled block scales; N % 16 == 0 <= 128, K % 256 == 0 <= 1024.
 * scale_path: 0 = block scales into TMEM by tcgen05.cp, 1 = through registers (tcgen05.st); anything else is rejected. The
 * arithmetic it checks is the reference GEMM of sm120fp4/reference.py:133-137. */
int b200moe_umma_probe(const void* a, const void* sfa, const void* b, const void* sfb, int N, int K, float* d,
                       int scale_path, int* status_dev, void* stream);

/* the same check for a CTA pair (tcgen05 cta_group::2: two SMs, one 256 x 128 x 64 MMA): a u8 [256, K/2], sfa 128x4-swizzled
 * over [256, K/16], b u8 [128, K/2], sfb 128x4-swizzled over [128, K/16], d f32 [256, 128], status_dev int32 [2]. */
int b200moe_umma_pair_probe(const void* a, const void* sfa, const void* b, const void* sfb, int K, float* d, int* status_dev,
                            void* stream);

/* HBM streaming floor of the kernels' access patterns, no math (the reference's k_stream probe,
 * sm120fp4/kernels/micro_floor.py:59-95): pattern 0 = 128-byte x box_rows TMA boxes from a row-major matrix of `pitch`
 * bytes per row, pattern 1 = contiguous tiles of tile_bytes by 1-D bulk copies; `stages` ring slots, `producers` issuing
 * threads per CTA, one CTA per SM. Time it with events around the call. */
int b200moe_stream_probe(const void* buf, long long bytes, int pattern, int pitch, int box_rows, int tile_bytes, int stages,
                         int producers, int* status_dev, void* stream);

/* W4A16 layer call for mid-sized batches (17 tokens up to a few hundred): the arithmetic of b200moe_decode_forward as a
 * grouped GEMM over per-expert gathered rows (four NVFP4 terms per token-expert pair), one pass over the touched experts'
 * weights instead of one per 16-token slice (the reference runs slices of 16, sm120fp4/vllm_backend.py:147-172). Needs
 * b200moe_layer_prepack and H, I <= 3072 (b200moe_mid_workspace_bytes returns the shape error otherwise); the workspace
 * (zeroed once) holds transient data of one call and can be shared by the layers of a stack. */
long long b200moe_mid_workspace_bytes(const b200moe_layer* layer, int max_tokens);
int b200moe_mid_forward(const b200moe_layer* layer, const void* x_bf16, const int* topk_ids, const float* topk_weights, int M,
                        void* out_bf16, void* workspace, long long workspace_bytes, int max_tokens, void* stream);
int b200moe_mid_status(const b200moe_layer* layer, const void* workspace, int max_tokens, void* stream);

/* expert-parallel fixed-capacity dispatch and combine (no counterpart in the reference: it declines expert parallelism,
 * sm120fp4/vllm_classes.py:46-47). dispatch: x bf16 [m, h], ids int32 [m, k] (global ids, negative = empty slot), wts f32
 * [m, k] -> per destination rank d a block of cap rows: token rows at dst_x[d] (bf16 [cap, h]; a row is stored only where d
 * owns one of its experts), the destination's local expert ids at dst_ids[d] (int32 [cap, k], -1 = not d's) and the routing
 * weights at dst_wts[d] (f32 [cap, k]). dst_x / dst_ids / dst_wts / dst_flag are HOST arrays of `world` device pointers: into
 * one packed send buffer (rows | ids | weights per destination - a single all-to-all then carries all three, and
 * b200moe_ep_unpack splits what arrived), or straight into the destination GPUs' receive arrays (plain peer stores over
 * NVLink); in that case dst_flag[d] is a counter in d's memory that is bumped once per row after the row is visible there,
 * and the destination waits with b200moe_ep_wait (bounded: a wait that runs out sets *status to 1 + the late peer's rank
 * and returns). b200moe_ep_return sends the partial rows back the same way. combine: y bf16 [world, cap, h] -> out bf16
 * [m, h], summed in rank order in fp32. */
int b200moe_ep_dispatch(const void* x, const int* ids, const float* wts, int m, int h, int k, int world, int experts_per_rank, int cap,
                        void* const* dst_x, int* const* dst_ids, float* const* dst_wts, unsigned* const* dst_flag, void* stream);
int b200moe_ep_unpack(const void* rbuf, long long block_bytes, int world, int cap, int h, int k, void* rx, int* rid, float* rw, void* stream);
int b200moe_ep_wait(const unsigned* flags, int world, int per_call, unsigned* calls, int* status, void* stream);
int b200moe_ep_return(const void* yl, int world, int cap, int h, int rank, void* const* back_y, unsigned* const* back_flag, void* stream);
int b200moe_ep_combine(const void* y, int m, int h, int world, int cap, void* out, void* stream);
/* The peer-store exchange in two launches per layer call instead of five: dispatch_wait = b200moe_ep_dispatch with counters +
 * the bounded wait for every peer's rows (flags_in: this rank's counters, one per peer; calls: device word, zeroed once, that
 * counts this rank's calls); return_combine = b200moe_ep_return + the bounded wait for the partial rows coming back
 * (flags_back) + b200moe_ep_combine over this rank's `back` array (bf16 [world, cap, h]). */
int b200moe_ep_dispatch_wait(const void* x, const int* ids, const float* wts, int m, int h, int k, int world, int experts_per_rank, int cap,
                             void* const* dst_x, int* const* dst_ids, float* const* dst_wts, unsigned* const* dst_flag,
                             const unsigned* flags_in, unsigned* calls, int* status, void* stream);
int b200moe_ep_return_combine(const void* yl, int world, int cap, int h, int rank, void* const* back_y, unsigned* const* back_flag,
                              const unsigned* flags_back, const unsigned* calls, int* status, const void* back, int m, void* out,
                              void* stream);

/* The peer-store exchange in its flagged-word form: every 8-byte store carries 4 bytes of payload and the call number, so
 * the sender never waits for its stores to be acknowledged across NVLink before it may signal (no system-scope fence, no
 * separate counters). Twice the bytes per row, one round trip less per exchange. peers_in / peers_back: host arrays of
 * `world` device pointers into the peers' flagged areas (entry d = where THIS rank's block starts at rank d); in / back:
 * this rank's own areas, in: uint2 [world][cap][h/2 + 2k], back: uint2 [world][cap][h/2] followed by `world` marker words;
 * both zeroed once. rx / rid / rw: the plain arrays the local layer call takes (bf16 [world*cap, h], int32 and f32
 * [world*cap, k]). calls: device uint32 [2], zeroed once; status: device int32, 0 or 1 + the rank whose words never arrived
 * within the bounded wait. A layer call is b200moe_ep_dispatch_ll, the local layer on (rx, rid, rw) -> yl,
 * b200moe_ep_return_combine_ll, in that order on one stream; cap and world are the same on every rank. A token row is sent
 * back only by the ranks that own one of its experts, and only those are waited for; a marker word per rank keeps a rank
 * from starting its next call before every peer has finished reading this one. No counterpart in the reference (it declines
 * expert parallelism, sm120fp4/vllm_classes.py:46-47). cap * world <= 1024 (B200MOE_ERR_LIMIT otherwise; the same holds
 * for b200moe_ep_return_combine): blocks of these kernels wait for blocks of the peers' kernels, so a grid must be resident
 * as a whole; larger blocks go through the stream-ordered exchange. */
int b200moe_ep_dispatch_ll(const void* x, const int* ids, const float* wts, int m, int h, int k, int world, int experts_per_rank, int cap,
                           void* const* peers_in, const void* in, void* rx, int* rid, float* rw, unsigned* calls, int* status, void* stream);
int b200moe_ep_return_combine_ll(const void* yl, const int* rid, int world, int cap, int h, int k, int rank, int experts_per_rank,
                                 void* const* peers_back, const void* back, const int* ids, int m, void* out, unsigned* calls, int* status,
                                 void* stream);
/* variable-size exchange (prefill batches; no counterpart in the reference either). plan: counts int32 [world], offsets int32
 * [world + 1], pos int32 [m, world] (row of token t in the send buffer for destination d, or -1), send_tok int32 [rows]
 * (destination-major, token order within a destination). gather: the rows of the send buffer (sx bf16 [rows, h], meta int32
 * [rows, 2k]); max_rows >= offsets[world] bounds the grid. combine_rows: out[t] = sum over destinations, in rank order, of
 * the partial row that came back for (t, d), fp32, one rounding. */
int b200moe_ep_plan(const int* ids, int m, int k, int world, int experts_per_rank, int* counts, int* offsets, int* pos, int* send_tok,
                    void* stream);
int b200moe_ep_gather(const void* x, const int* ids, const float* wts, const int* send_tok, const int* offsets, int h, int k, int world,
                      int experts_per_rank, int max_rows, void* sx, int* meta, void* stream);
int b200moe_ep_combine_rows(const void* back, const int* pos, int m, int h, int world, void* out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H */
