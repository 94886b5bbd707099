/*
 * b200moe -- C ABI of the B200 (sm_100a) NVFP4 sparse-MoE block.
 *
 * Conventions (the ones the reference's own native libraries use, kernels/nvfp4-moe/src/
 * qwen36_nvfp4_bitexact.cu:30-42,731-740 and kernels/decode-moe/src/qwen_moe_decode.cu:272-303):
 *   - plain C symbols, raw device pointers, sizes and strides; `stream` is a cudaStream_t;
 *   - every launch function validates its arguments on the host first and returns 0, a positive
 *     cudaError_t, or a negative B200MOE_E_* code; on a non-zero return nothing was launched;
 *   - nothing here allocates, frees or synchronises; scratch memory is passed in by the caller
 *     (sizes from the *_workspace_bytes helpers);
 *   - the probes (abi_version, build_id, error_string, *_workspace_bytes) need no CUDA context.
 *
 * NVFP4 bank record of one expert (freetoken/python/freetoken/layers/quantization/moe/nvfp4.py:53-62):
 *   gate_up [2I, H/2] u8 (two E2M1 codes per byte, low nibble = even k), gate_up_scale [2I, H/16] e4m3,
 *   gate_up_global [2I] f32, down [H, I/2] u8, down_scale [H, I/16] e4m3, down_global [H] f32.
 *   W[n,k] = E2M1[code] * e4m3(scale[n,k/16]) * global[n]; rows [0,I) of gate_up are gate, [I,2I) up.
 */
#ifndef B200MOE_H_
#define B200MOE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200MOE_ABI_VERSION 1

enum {
  B200MOE_OK = 0,
  B200MOE_E_NULL = -1,      /* a required pointer is null */
  B200MOE_E_SHAPE = -2,     /* a size is outside what the kernels support */
  B200MOE_E_ALIGN = -3,     /* a pointer or stride breaks the 16-byte rule */
  B200MOE_E_WORKSPACE = -4, /* workspace too small */
  B200MOE_E_DEVICE = -5,    /* the current device is not sm_100 */
  B200MOE_E_STATIC_LIMIT = -6 /* the call needs more scratch than the built-in static array holds */
};

/* Probes.  Replace qwen_moe_decode_abi_version / qwen_nvfp4_build_id / qwen_nvfp4_cuda_error
 * (kernels/decode-moe/src/qwen_moe_decode.cu:272-276, kernels/nvfp4-moe/src/qwen36_nvfp4_bitexact.cu:801-810). */
int b200moe_abi_version(void);
const char* b200moe_build_id(void);
const char* b200moe_error_string(int code);

/* ---- host banks ---------------------------------------------------------------------------------
 * Pin-after-fill for the host expert banks: register an already filled, page-aligned host buffer as portable +
 * mapped, and look up the address a kernel must use to read it (equal to the host address under unified
 * addressing).  Replaces host_register / host_device_ptr of the reference's pinned-memory extension
 * (freetoken/python/freetoken/kernel/pinned.py:52-68; used by freetoken/python/freetoken/moe/host_banks.py:137-151). */
int b200moe_host_register(void* addr, int64_t nbytes);
int b200moe_host_unregister(void* addr);
int b200moe_host_device_ptr(void* host_addr, void** device_addr);

/* ---- router: fp32 softmax + top-k + renormalise ------------------------------------------------
 * Replaces fused_topk_softmax (freetoken/python/freetoken/kernel/triton/moe_router.py:109-157).
 * logits [T, E] bf16 (dtype 0) or f32 (dtype 1), row stride in elements; E <= 512.
 * Ties: higher logit first, then the LOWER expert id.  `limit` (device int32 or int64 scalar, may be
 * null): rows >= *limit get id -1.  weights [T, top_k] f32, ids [T, top_k] i32, selection order. */
int b200moe_router_topk(const void* logits, int logits_dtype, int64_t row_stride, int T, int E, int top_k,
                        int renormalize, const void* limit, int limit_is_i64, float* weights, int32_t* ids,
                        void* stream);

/* ---- permutation ------------------------------------------------------------------------------
 * Replaces moe_align_block_size (freetoken/python/freetoken/moe/fused.py:47-117, kernel
 * freetoken/python/freetoken/kernel/triton/moe_align.py:216-325) with a DETERMINISTIC order: inside an
 * expert, flat route ids (t*top_k+k) ascend.  ids in [0, num_experts] are counted (the reference's
 * effective_E = num_experts + 1); others are dropped.
 * Outputs (any may be null except counts/offsets):
 *   sorted_token_ids [cap]  padded per expert to `block`, unwritten = numel      (reference layout)
 *   expert_ids [cap/block]  expert of each block, -1 past the end               (reference layout)
 *   num_tokens_post_pad [1]
 *   sorted_routes [numel]   unpadded route ids in (expert, route) order
 *   expert_offsets [num_experts + 2]  exclusive prefix of the per-expert counts (unpadded) */
int64_t b200moe_permute_workspace_bytes(int numel, int num_experts);
int b200moe_permute(const int32_t* topk_ids, int numel, int num_experts, int block, int32_t* sorted_token_ids,
                    int sorted_cap, int32_t* expert_ids, int expert_ids_cap, int32_t* num_tokens_post_pad,
                    int32_t* sorted_routes, int32_t* expert_offsets, void* workspace, int64_t workspace_bytes,
                    void* stream);

/* ---- expert-slot cache -------------------------------------------------------------------------
 * State (freetoken/python/freetoken/moe/offload_cache.py:205-227): slot_for_id [L*E] i32 (-1 absent),
 * id_of_slot [S] i32 (flat id layer*E+expert), usage [S] i64, step [1] i64.
 * slot_ensure replaces flashlib lru_ensure as called from freetoken/python/freetoken/moe/offload_kernels.py:19-40:
 * step += 1; hits get usage = step; DISTINCT misses in ascending id take victims in ascending
 * (usage, slot) among slots untouched by this call; plan -> src_indices (layer-local expert id),
 * evict_slots, num_indices; ids_out (may alias ids) = slot ids; stats (null or i64[3]) += (active, missing, 1).
 * The *_host twin runs the same policy on host arrays (for callers that plan copies on the CPU). */
typedef struct {
  int32_t* slot_for_id;
  int32_t* id_of_slot;
  int64_t* usage;
  int64_t* step;
  int32_t* src_indices; /* [>= min(n_ids, S)] */
  int32_t* evict_slots; /* [>= min(n_ids, S)] */
  int64_t* num_indices; /* [1] */
  int64_t* stats;       /* null or [3] of this layer */
  int32_t num_layers, num_experts, cache_size;
} b200moe_slot_tables;

int b200moe_slot_reset(const b200moe_slot_tables* t, void* stream);
int b200moe_slot_ensure(const b200moe_slot_tables* t, int layer, const int32_t* ids, int n_ids, int32_t* ids_out,
                        void* stream);
int b200moe_slot_ensure_host(const b200moe_slot_tables* t, int layer, const int32_t* ids, int n_ids,
                             int32_t* ids_out);
/* Prefill through the cache: split the experts a chunk routes to (or the whole layer: select_all) into residents
 * (slot >= first_lru_slot, gathered device-to-device) and misses (fetched from the host bank), both as (buffer row,
 * source) lists in ascending expert id with counts[2] = {hits, misses}; buffer row = buffer_row0 + expert id.
 * Replaces mark_selected + prefill_split_compact (freetoken/python/freetoken/moe/offload_kernels.py:63-113) as used by
 * freetoken/python/freetoken/moe/offload_cache.py:1046-1121,1160-1200.  The lists feed b200moe_slot_gather. */
int b200moe_prefill_split(const int32_t* topk_ids, int n_ids, const int32_t* slot_row, int num_experts, int first_lru_slot,
                          int buffer_row0, int select_all, int32_t* hit_dst, int32_t* hit_src, int32_t* miss_dst,
                          int32_t* miss_src, int64_t* counts, void* stream);
/* One-layer-ahead speculative prefetch (freetoken/python/freetoken/moe/pregate.py:77-117,197-212): the next layer's
 * router applied to its post-attention RMSNorm of the residual row (one token), then the first `cap` of the top_k
 * predictions (score order, ties lower id) that are not resident, padded to `width` with the first of them (with
 * the top-1 prediction when none misses).  logits [E] f32 and query [width] i32 are outputs; the caller hands
 * `query` to b200moe_slot_ensure and gathers the plan on a side stream. */
int b200moe_pregate_predict(const void* residual, const void* norm_w, float eps, const void* gate_w, int64_t gate_stride,
                            int hidden, int num_experts, const int32_t* slot_row, int cap, int top_k, float* logits,
                            int32_t* query, int width, void* stream);
/* whole layer into slots [0,E), position == expert id (offload_kernels.py:296-332). */
int b200moe_slot_materialize(const b200moe_slot_tables* t, int layer, void* stream);

/* Miss fills.  copy_missing / copy_planned (offload_cache.py:1471-1533):
 *   for bank b, i < n: dst[b] + evict_slots[i]*row_bytes[b]  <-  src[b] + src_indices[i]*row_bytes[b]
 * slot_fill: plan on the HOST, one cudaMemcpyAsync per (miss, bank) on `stream` (a copy stream);
 *   replaces the batched-memcpy transport of freetoken/python/freetoken/kernel/csrc/jit/batch_memcpy.cuh:16-58.
 * slot_gather: plan on the DEVICE (num_indices is a device scalar, so the launch is fixed-shape and
 *   graph-capturable); sources may be mapped pinned host memory or device memory; replaces
 *   fast_index_copy_multi (freetoken/python/freetoken/kernel/csrc/jit/fast_index_copy.cuh:486-512). */
int b200moe_slot_fill(int num_banks, void* const* dst_banks, const void* const* src_banks,
                      const int64_t* row_bytes, const int32_t* evict_slots_host,
                      const int32_t* src_indices_host, int n, void* stream);
int b200moe_slot_gather(int num_banks, void* const* dst_banks_dev, const void* const* src_banks_dev,
                        const int64_t* row_bytes_dev, const int32_t* evict_slots, const int32_t* src_indices,
                        const int64_t* num_indices, int max_rows, int blocks_per_bank, void* stream);

/* ---- expert banks ------------------------------------------------------------------------------ */
typedef struct {
  const uint8_t* gate_up;        /* [S, 2I, H/2] */
  const uint8_t* gate_up_scale;  /* [S, 2I, H/16] e4m3 */
  const float* gate_up_global;   /* [S, 2I] */
  const uint8_t* down;           /* [S, H, I/2] */
  const uint8_t* down_scale;     /* [S, H, I/16] */
  const float* down_global;      /* [S, H] */
  int32_t num_slots, hidden, intermediate;
  /* Bytes from one slot to the next, per role in the order above; 0 = dense ([S, ...] contiguous).  A non-zero
   * stride lets the six roles of a slot live in ONE contiguous record (slot s of every role inside
   * [s*record, (s+1)*record)), so that a miss fill is a single copy.  Multiples of 16. */
  int64_t slot_stride[6];
} b200moe_banks;

typedef struct {
  const void* router_w;       /* [E, H] bf16 */
  const void* shared_gate_up; /* [2*SI, H] bf16 */
  const void* shared_down;    /* [H, SI] bf16 */
  const void* shared_gate;    /* [1, H] bf16 */
  int32_t num_experts, shared_intermediate;
} b200moe_dense;

/* ---- decode (1..8 tokens) ---------------------------------------------------------------------
 * decode_experts replaces the routed-expert body _fused_experts_decode_nvfp4
 * (freetoken/python/freetoken/moe/fused_nvfp4.py:140-179: gemm1 -> act -> gemm2 * weight -> sum over k)
 * and the C entry qwen_moe_decode_gemv (kernels/decode-moe/src/qwen_moe_decode.cu:277-293).
 * x [M,H] bf16, topk_ids [M,top_k] i32 = rows of the banks (slot ids; <0 = skipped route),
 * topk_weights [M,top_k] f32, out [M,H] bf16.  workspace: b200moe_decode_workspace_bytes. */
int64_t b200moe_decode_workspace_bytes(int M, int top_k, int hidden, int intermediate, int shared_intermediate,
                                       int num_experts);
int b200moe_decode_experts(const void* x, const b200moe_banks* banks, const float* topk_weights,
                           const int32_t* topk_ids, int M, int top_k, void* out, void* workspace,
                           int64_t workspace_bytes, void* stream);
/* No counterpart in the reference.  b200moe_decode_experts for callers that cannot allocate device memory
 * (a plugin host that forbids cudaMalloc after start-up, code running while the allocator is locked, a
 * process that owns no allocator): same inputs, outputs and results, but the intermediate activations live
 * in a static device array of B200MOE_STATIC_SCRATCH_BYTES inside the library, held by every GPU that loads
 * it.  Returns B200MOE_E_STATIC_LIMIT when M * top_k * intermediate does not fit.  The first call on a device
 * resolves the array's address and should come before any stream capture.  All calls share the array: calls
 * that overlap on the GPU race, so keep them ordered.  Allocates nothing. */
#define B200MOE_STATIC_SCRATCH_BYTES (512 * 1024)
int b200moe_decode_experts_static(const void* x, const b200moe_banks* banks, const float* topk_weights,
                                  const int32_t* topk_ids, int M, int top_k, void* out, void* stream);

/* Stage A of the whole block Qwen3_5MoE.forward (freetoken/python/freetoken/models/qwen3_5_moe/moe.py:77-106):
 * router logits (bf16), shared gate_up, shared gate logit, then router top-k.  Writes logits [M,E] bf16,
 * topk_weights, topk_ids (expert ids; the caller may run slot_ensure on them before stage B). */
int b200moe_decode_block_route(const void* x, const b200moe_dense* dense, int M, int hidden, int top_k,
                               void* logits_out, float* topk_weights, int32_t* topk_ids, void* workspace,
                               int64_t workspace_bytes, void* stream);
/* Stage B: routed experts + shared expert + merge  out = bf16(routed + bf16(shared * bf16(sigmoid(g)))). */
/* The dense rows of a decode layer by segment (bit 0: router logits -> logits_out [M, E] bf16; bit 1: shared
 * gate_up -> workspace; bit 2: shared gate logit -> workspace).  Lets a caller run the router first, hand the ids
 * to the slot cache, and compute the shared expert's rows while the miss fills run on another stream
 * (freetoken/python/freetoken/decode_overlap.py:44-59, freetoken/python/freetoken/layers/moe.py:286-302). */
int b200moe_decode_dense_rows(const void* x, const b200moe_dense* dense, int M, int hidden, int segment_mask,
                              void* logits_out, void* workspace, int64_t workspace_bytes, void* stream);
int b200moe_decode_block_experts(const void* x, const b200moe_banks* banks, const b200moe_dense* dense,
                                 const float* topk_weights, const int32_t* topk_ids, int M, int top_k, void* out,
                                 void* workspace, int64_t workspace_bytes, void* stream);

/* The whole block in three launches (all experts resident: ids are expert ids == bank rows): dense rows, then
 * GEMM1 with the router's top-k in its prologue (it also writes topk_weights / topk_ids), then GEMM2 + merge. */
int b200moe_decode_block(const void* x, const b200moe_banks* banks, const b200moe_dense* dense, int M, int top_k,
                         void* logits_out, float* topk_weights, int32_t* topk_ids, void* out, void* workspace,
                         int64_t workspace_bytes, void* stream);
/* Programmatic dependent launch between the decode kernels (default on); measurement knob, no counterpart in the
 * reference. */
int b200moe_set_pdl(int enable);

/* One decode step (M tokens) over a stack of layers served from the slot cache, planned on the host.  Per layer:
 * LRU on host tables, one cudaMemcpyAsync per (miss, bank) on `copy_stream`, event hand-over, then the decode
 * launches on `compute_stream` with slot ids; a fill only overwrites slots no pending kernel reads (it waits for the
 * compute of `lookahead` layers earlier, 1 <= lookahead <= 64; a layer without misses waits for nothing and records
 * no fill event).  The driver loop of the reference lives in Python
 * (freetoken/python/freetoken/layers/moe.py:286-339 with offload_cache.py:1288-1302,1471-1533); this is its native form.
 * create/destroy own the CUDA events; the step call allocates nothing on the device and never blocks on the GPU.
 *   host_tables->stats, when not null, is [L, 3] (one row per layer);
 *   routing_host [L, M, top_k] expert ids; slots_host_pinned / slots_dev [L, M, top_k] receive the slot ids:
 *   the call writes slots_host_pinned on the host and enqueues an asynchronous copy from it, so the buffer must
 *   stay untouched until that copy has run on `compute_stream` (give every step in flight its own buffer);
 *   weights_dev: router weights [M, top_k] per layer (stride in elements, 0 = shared by all layers);
 *   dense: array of per-layer dense weights (stride in bytes, 0 = shared); out: [M, H] per layer (stride in bytes);
 *   miss_src / miss_dst [L, M*top_k] and miss_count [L] (may be null) receive the ordered miss plan. */
typedef struct b200moe_offload b200moe_offload;
b200moe_offload* b200moe_offload_create(const b200moe_slot_tables* host_tables, int num_banks, void* const* dst_banks,
                                        const void* const* src_banks /* [L * num_banks] */, const int64_t* row_bytes,
                                        int lookahead, int* err);
void b200moe_offload_destroy(b200moe_offload* o);
int b200moe_offload_decode_step(b200moe_offload* o, const int32_t* routing_host, int M, int top_k,
                                int32_t* slots_host_pinned, int32_t* slots_dev, const float* weights_dev,
                                int64_t weights_layer_stride, const void* x, const b200moe_banks* cache,
                                const b200moe_dense* dense, int64_t dense_layer_stride, void* out,
                                int64_t out_layer_stride, void* workspace, int64_t workspace_bytes, int32_t* miss_src,
                                int32_t* miss_dst, int32_t* miss_count, int64_t* h2d_bytes, void* copy_stream,
                                void* compute_stream);

/* ---- prefill (grouped GEMM on tcgen05) ----------------------------------------------------------
 * Replaces fused_experts_nvfp4 (freetoken/python/freetoken/moe/fused_nvfp4.py:287-333) and the C entry
 * qwen_nvfp4_prefill (kernels/nvfp4-moe/src/qwen36_nvfp4_bitexact.cu:731-740).  topk_ids are rows of the
 * banks (raw expert ids of a whole-layer view).  out [T,H] bf16 may alias x.  If `shared`/`shared_gate_logit`
 * are non-null ([T,H] bf16, [T,1] bf16) the merge of moe.py:95-97 is fused into the final sum. */
int64_t b200moe_prefill_workspace_bytes(int T, int top_k, int hidden, int intermediate, int num_slots);
int b200moe_prefill_experts(const void* x, const b200moe_banks* banks, const float* topk_weights,
                            const int32_t* topk_ids, int T, int top_k, const void* shared,
                            const void* shared_gate_logit, void* out, void* workspace, int64_t workspace_bytes,
                            int32_t* status /* device int[4], zeroed by the call; [0] != 0 = a bounded wait gave up */,
                            void* stream);

/* The same call cut into its stages (bit mask), so that a benchmark can time each kernel on its own stream
 * with events.  Stages read what earlier stages left in the workspace; B200MOE_STAGE_ALL == prefill_experts. */
enum {
  B200MOE_STAGE_PLAN = 1,    /* permutation + tile list */
  B200MOE_STAGE_GEMM1 = 2,   /* gate_up grouped GEMM + SwiGLU */
  B200MOE_STAGE_GEMM2 = 4,   /* down grouped GEMM * router weight */
  B200MOE_STAGE_COMBINE = 8, /* sum over routes (+ merge) */
  B200MOE_STAGE_ALL = 15,
  B200MOE_STAGE_ROUTE_ORDER = 16 /* modifier: leave the per-route rows [T, top_k, hidden] in route order in the workspace
                                    (for a caller that reads them); without it they sit in expert order and only the
                                    combine stage, given the same modifier state, can use them */
};
int b200moe_prefill_stages(const void* x, const b200moe_banks* banks, const float* topk_weights,
                           const int32_t* topk_ids, int T, int top_k, const void* shared,
                           const void* shared_gate_logit, void* out, void* workspace, int64_t workspace_bytes,
                           int32_t* status, int stage_mask, void* stream);

/* ---- small fused element-wise ops ---------------------------------------------------------------
 * silu_and_mul: out[r, d] = bf16(silu(f32 in[r, d]) * f32 in[r, D + d])  (freetoken/python/freetoken/layers/activation.py:71-83)
 * shared_epilogue: out = bf16(routed + bf16(shared * bf16(sigmoid(gate))))  (freetoken/python/freetoken/moe/shared_epilogue.py:40-63)
 * sum_routes: out[t] = bf16(sum_k f32(in[t,k]))  (freetoken/python/freetoken/kernel/triton/fused_moe.py:112-153) */
int b200moe_silu_and_mul(const void* in, void* out, int rows, int D, void* stream);
int b200moe_shared_epilogue(const void* routed, const void* shared, const void* gate, void* out, int T, int H,
                            void* stream);
int b200moe_sum_routes(const void* in, void* out, int T, int top_k, int H, void* stream);
/* The decoder layer's glue around the block: residual add fused with the RMSNorm that feeds it
 * (freetoken/python/freetoken/models/qwen3_5_moe/model.py:63-77; kernel semantics of
 * freetoken/python/freetoken/kernel/triton/norm.py:44-111): z = f32(x) + f32(residual); residual = bf16(z);
 * x = bf16(z * rsqrt(mean(z^2) + eps) * (w + plus_one)).  rmsnorm is the form without a residual (out-of-place). */
int b200moe_fused_add_rmsnorm(void* x, void* residual, const void* weight, float eps, int plus_one, int64_t rows, int H,
                              void* stream);
int b200moe_rmsnorm(const void* x, const void* weight, void* out, float eps, int plus_one, int64_t rows, int H,
                    void* stream);
/* The block's dense bf16 linears on the tensor cores (tcgen05): the router's gate and the shared expert's projections
 * (freetoken/python/freetoken/models/qwen3_5_moe/moe.py:20-36,66,86,99-106; the reference calls a library GEMM,
 * freetoken/python/freetoken/layers/quantization/linear/unquantized.py:18-24).
 *   swiglu == 0: out[T, N] = bf16(x[T, K] . w[N, K]^T + bias[N])        bias fp32 or null; N % 8 == 0
 *   swiglu == 1: w = [2 * N/2, K] (gate rows, then up rows); out[T, N/2] = bf16(silu(bf16(gate)) * bf16(up)), the
 *                result of the linear followed by the activation kernel; (N/2) % 64 == 0
 * K % 64 == 0; x, w, out 16-byte aligned and contiguous.  status: one int32 on the device, set non-zero if a wait
 * inside the kernel ran out (never in a correct run); the caller zeroes it once.
 * row_dot: out[T] = bf16(x[T, K] . w[K]) -- the shared expert's scalar gate logit (K % 8 == 0). */
int b200moe_dense_linear(const void* x, const void* w, const float* bias, void* out, int T, int N, int K, int swiglu,
                         int32_t* status, void* stream);
int b200moe_row_dot(const void* x, const void* w, void* out, int T, int K, void* stream);
/* sum_routes that skips routes whose id is outside [0, num_slots) (topk_ids may be null = keep all) and can
 * fuse the merge with the shared expert; used by expert-parallel prefill after the per-route rows came back
 * from their owners (no counterpart in the reference, which has no expert parallelism). */
int b200moe_combine_routes(const void* ic3, const int32_t* topk_ids, int num_slots, int T, int top_k, int H,
                           const void* shared, const void* shared_gate_logit, void* out, void* stream);
/* Expert-parallel prefill, the part that runs on the expert's owner (no counterpart in the reference, which has
 * no expert parallelism): the two grouped GEMMs over a slice of the box's tokens (x [T, H], already in local
 * memory; its rows are global tokens first_token, first_token + 1, ... modulo world * tokens_per_rank, so a slice
 * may run from the last rank's tokens into the first's; global token g lives on rank g / tokens_per_rank) for the
 * routes whose expert lives here (local_ids [T, top_k]: local expert id, or -1).  The second GEMM's epilogue
 * stores every per-route row DIRECTLY into the ic3 buffer of the token's home GPU (peer_ic3: device array of
 * `world` pointers to [tokens_per_rank*top_k, H] bf16, peer-mapped) -- the combine exchange is fused into the
 * kernel; the caller then runs a cross-GPU barrier and b200moe_combine_routes.  Calling it for a few groups of
 * source ranks lets the copies of the later groups' tokens overlap the GEMMs of the tokens that are already here. */
int b200moe_prefill_ep_routes(const void* x, const b200moe_banks* local_banks, const float* weights,
                              const int32_t* local_ids, int T, int first_token, int top_k, void* const* peer_ic3,
                              int world, int tokens_per_rank, void* workspace, int64_t workspace_bytes,
                              int32_t* status, void* stream);
/* Byte offset of the per-route output rows ic3 [T*top_k, H] bf16 inside the prefill workspace (valid after
 * stages PLAN|GEMM1|GEMM2).  Rows of dropped routes are not written. */
int64_t b200moe_prefill_ic3_offset(int T, int top_k, int hidden, int intermediate, int num_slots);

#ifdef __cplusplus
}
#endif
#endif /* B200MOE_H_ */
