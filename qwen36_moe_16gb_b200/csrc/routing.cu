// Router (fp32 softmax + top-k with the lowest-id tie rule) and the deterministic token permutation.
#include "common.cuh"
#include "router.cuh"

namespace b200moe {

// ------------------------------------------------------------------------------------------------
// Router: one warp per token; lane j owns experts j, j+32, ...  (coalesced row read).
// ------------------------------------------------------------------------------------------------
template <int NPL, typename LogitT>
__global__ void __launch_bounds__(128) router_topk_kernel(const LogitT* __restrict__ logits, int64_t row_stride, int T,
                                                          int E, int top_k, int renormalize, const void* limit_ptr,
                                                          int limit_is_i64, float* __restrict__ weights,
                                                          int32_t* __restrict__ ids) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  const LogitT* src = logits + (int64_t)row * row_stride;

  router_select<NPL, LogitT>(src, E, top_k, renormalize, lane, weights + (int64_t)row * top_k, ids + (int64_t)row * top_k);
  if (limit_ptr != nullptr) {
    const long long lim = limit_is_i64 ? *reinterpret_cast<const long long*>(limit_ptr)
                                       : (long long)*reinterpret_cast<const int*>(limit_ptr);
    if (row >= lim)
      for (int kk = lane; kk < top_k; kk += 32) ids[(int64_t)row * top_k + kk] = -1;
  }
}

template <typename LogitT>
static int launch_router(const void* logits, int64_t stride, int T, int E, int top_k, int renorm, const void* limit,
                         int limit_is_i64, float* w, int32_t* ids, cudaStream_t st) {
  const int warps = 4;
  dim3 grid((T + warps - 1) / warps), block(warps * 32);
  const LogitT* l = reinterpret_cast<const LogitT*>(logits);
  const int npl = (E + 31) / 32;
#define B200MOE_ROUTER_CASE(N)                                                                                     \
  if (npl <= N) {                                                                                                  \
    router_topk_kernel<N, LogitT><<<grid, block, 0, st>>>(l, stride, T, E, top_k, renorm, limit, limit_is_i64, w, ids); \
    return check_launch();                                                                                         \
  }
  B200MOE_ROUTER_CASE(1)
  B200MOE_ROUTER_CASE(2)
  B200MOE_ROUTER_CASE(4)
  B200MOE_ROUTER_CASE(8)
  B200MOE_ROUTER_CASE(16)
#undef B200MOE_ROUTER_CASE
  return B200MOE_E_SHAPE;
}

// ------------------------------------------------------------------------------------------------
// Permutation.  Routes are cut into segments of SEG consecutive flat route ids, one warp each.
//   K1 count   : per-segment histogram -> seg_counts[seg][E1]; also fills the padded list with the sentinel
//   K2 segscan : one CTA per expert: exclusive scan of its column over the segments, total -> counts[e]
//   K3 experts : one CTA: padded / unpadded prefix sums, expert_ids, num_tokens_post_pad
//   K4 scatter : each warp replays its segment in route order -> stable positions
// ------------------------------------------------------------------------------------------------
constexpr int SEG = 128;          // routes per warp
constexpr int PERM_WARPS = 8;     // warps per CTA

__global__ void __launch_bounds__(PERM_WARPS * 32) perm_count_kernel(const int32_t* __restrict__ ids, int numel, int E1,
                                                                     int nseg, int32_t* __restrict__ seg_counts,
                                                                     int32_t* __restrict__ sorted_token_ids,
                                                                     int sorted_cap) {
  extern __shared__ int32_t sm_counts[];  // [PERM_WARPS][E1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < PERM_WARPS * E1; i += blockDim.x) sm_counts[i] = 0;
  if (sorted_token_ids != nullptr)
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < sorted_cap; i += gridDim.x * blockDim.x)
      sorted_token_ids[i] = numel;
  __syncthreads();
  const int seg = blockIdx.x * PERM_WARPS + warp;
  if (seg < nseg) {
    int32_t* mine = sm_counts + warp * E1;
    int id[SEG / 32];  // all loads of the segment in flight before the first one is used
#pragma unroll
    for (int it = 0; it < SEG / 32; ++it) {
      const int r = seg * SEG + it * 32 + lane;
      id[it] = r < numel ? ids[r] : -1;
    }
#pragma unroll
    for (int it = 0; it < SEG / 32; ++it)
      if (id[it] >= 0 && id[it] < E1) atomicAdd(&mine[id[it]], 1);
    __syncwarp();
    for (int e = lane; e < E1; e += 32) seg_counts[(int64_t)seg * E1 + e] = mine[e];
  }
}

__global__ void __launch_bounds__(256) perm_segscan_kernel(int32_t* __restrict__ seg_counts, int nseg, int E1,
                                                           int32_t* __restrict__ counts) {
  // exclusive scan of column e over segments, in place
  __shared__ int32_t warp_tot[8];
  __shared__ int32_t carry_s;
  const int e = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < nseg; base += 256) {
    const int s = base + threadIdx.x;
    const int v = s < nseg ? seg_counts[(int64_t)s * E1 + e] : 0;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int woff = 0;
    for (int w = 0; w < warp; ++w) woff += warp_tot[w];
    const int carry = carry_s;
    if (s < nseg) seg_counts[(int64_t)s * E1 + e] = carry + woff + incl - v;
    __syncthreads();
    if (threadIdx.x == 255) carry_s = carry + woff + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0) counts[e] = carry_s;
}

__global__ void __launch_bounds__(1024) perm_experts_kernel(const int32_t* __restrict__ counts, int E1, int block,
                                                            int32_t* __restrict__ padded_off,  // [E1+1] workspace
                                                            int32_t* __restrict__ expert_offsets,  // [E1+1]
                                                            int32_t* __restrict__ expert_ids, int expert_ids_cap,
                                                            int32_t* __restrict__ num_tokens_post_pad) {
  // E1 <= 1025: thread e scans expert e's padded and plain counts (warp shuffles, then the warp totals); the
  // totals land in slot E1.  All threads then fill expert_ids.
  __shared__ int32_t total_pad;
  __shared__ int32_t wpad[32], wcnt[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int carry_p = 0, carry_u = 0;
  for (int base = 0; base < E1; base += 1024) {  // one pass unless E1 == 1025
    const int e = base + threadIdx.x;
    const int c = e < E1 ? counts[e] : 0;
    const int pc = (c + block - 1) / block * block;
    int sp = pc, su = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int a = __shfl_up_sync(0xffffffffu, sp, o), b = __shfl_up_sync(0xffffffffu, su, o);
      if (lane >= o) {
        sp += a;
        su += b;
      }
    }
    if (lane == 31) {
      wpad[warp] = sp;
      wcnt[warp] = su;
    }
    __syncthreads();
    int bp = carry_p, bu = carry_u, tp = carry_p, tu = carry_u;
    for (int w = 0; w < 32; ++w) {
      if (w < warp) {
        bp += wpad[w];
        bu += wcnt[w];
      }
      tp += wpad[w];
      tu += wcnt[w];
    }
    if (e < E1) {
      padded_off[e] = bp + sp - pc;
      expert_offsets[e] = bu + su - c;
    }
    carry_p = tp;
    carry_u = tu;
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    padded_off[E1] = carry_p;
    expert_offsets[E1] = carry_u;
    total_pad = carry_p;
    if (num_tokens_post_pad != nullptr) *num_tokens_post_pad = carry_p;
  }
  __syncthreads();
  if (expert_ids != nullptr) {
    for (int b = threadIdx.x; b < expert_ids_cap; b += blockDim.x) {
      const int pos = b * block;
      int v = -1;
      if (pos < total_pad) {
        int lo = 0, hi = E1;  // last e with padded_off[e] <= pos
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (padded_off[mid] <= pos) lo = mid; else hi = mid;
        }
        v = lo;
      }
      expert_ids[b] = v;
    }
  }
}

__global__ void __launch_bounds__(PERM_WARPS * 32) perm_scatter_kernel(const int32_t* __restrict__ ids, int numel, int E1,
                                                                       int nseg, const int32_t* __restrict__ seg_prefix,
                                                                       const int32_t* __restrict__ padded_off,
                                                                       const int32_t* __restrict__ expert_offsets,
                                                                       int32_t* __restrict__ sorted_token_ids,
                                                                       int32_t* __restrict__ sorted_routes,
                                                                       int32_t* __restrict__ inv_routes) {
  extern __shared__ int32_t sm_run[];  // [PERM_WARPS][E1] running rank inside the expert
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seg = blockIdx.x * PERM_WARPS + warp;
  if (seg >= nseg) return;
  int32_t* run = sm_run + warp * E1;
  int idr[SEG / 32];  // the segment's ids: loaded together, ahead of the prefix row
#pragma unroll
  for (int it = 0; it < SEG / 32; ++it) {
    const int r = seg * SEG + it * 32 + lane;
    idr[it] = r < numel ? ids[r] : -1;
  }
  // run[e] = routes of expert e in earlier segments; it grows as this segment's routes are placed
  for (int e = lane; e < E1; e += 32) run[e] = seg_prefix[(int64_t)seg * E1 + e];
  __syncwarp();
#pragma unroll
  for (int it = 0; it < SEG / 32; ++it) {
    const int r = seg * SEG + it * 32 + lane;
    int id = idr[it];
    if (id < 0 || id >= E1) id = -1;
    const unsigned key = id >= 0 ? (unsigned)id : 0x40000000u + lane;  // invalid routes never match
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    int rank = 0;
    if (id >= 0) rank = run[id] + __popc(peers & ((1u << lane) - 1u));
    __syncwarp();
    if (id >= 0 && (peers & ((1u << lane) - 1u)) == 0) run[id] += __popc(peers);
    __syncwarp();
    if (id >= 0) {
      if (sorted_token_ids != nullptr) sorted_token_ids[padded_off[id] + rank] = r;
      if (sorted_routes != nullptr) sorted_routes[expert_offsets[id] + rank] = r;
    }
    // inverse of sorted_routes: route -> sorted position, -1 for a route without a valid expert
    if (inv_routes != nullptr && r < numel) inv_routes[r] = id >= 0 ? expert_offsets[id] + rank : -1;
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_router_topk(const void* logits, int logits_dtype, int64_t row_stride, int T, int E, int top_k,
                                   int renormalize, const void* limit, int limit_is_i64, float* weights, int32_t* ids,
                                   void* stream) {
  if (T == 0) return 0;
  if (!logits || !weights || !ids) return B200MOE_E_NULL;
  if (T < 0 || E < 1 || E > 512 || top_k < 1 || top_k > E || row_stride < E) return B200MOE_E_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (logits_dtype == 0) return launch_router<__nv_bfloat16>(logits, row_stride, T, E, top_k, renormalize, limit, limit_is_i64, weights, ids, st);
  if (logits_dtype == 1) return launch_router<float>(logits, row_stride, T, E, top_k, renormalize, limit, limit_is_i64, weights, ids, st);
  return B200MOE_E_SHAPE;
}

extern "C" int64_t b200moe_permute_workspace_bytes(int numel, int num_experts) {
  if (numel < 0 || num_experts < 1) return 0;
  const int64_t e1 = num_experts + 1;
  const int64_t nseg = (numel + SEG - 1) / SEG;
  // seg_counts [nseg][E1] + counts [E1] + padded_off [E1+1]
  return (nseg * e1 + e1 + e1 + 1 + 8) * 4;
}

namespace b200moe {
int permute_with_inverse(const int32_t* topk_ids, int numel, int num_experts, int block, int32_t* sorted_token_ids,
                         int sorted_cap, int32_t* expert_ids, int expert_ids_cap, int32_t* num_tokens_post_pad,
                         int32_t* sorted_routes, int32_t* expert_offsets, int32_t* inv_routes, void* workspace,
                         int64_t workspace_bytes, void* stream) {
  if (!expert_offsets || !workspace || (numel > 0 && !topk_ids)) return B200MOE_E_NULL;
  if (numel < 0 || num_experts < 1 || num_experts > 1024 || block < 1) return B200MOE_E_SHAPE;
  if (sorted_token_ids && sorted_cap < 0) return B200MOE_E_SHAPE;
  if (workspace_bytes < b200moe_permute_workspace_bytes(numel, num_experts)) return B200MOE_E_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int E1 = num_experts + 1;
  const int nseg = (numel + SEG - 1) / SEG;
  int32_t* seg_counts = reinterpret_cast<int32_t*>(workspace);
  int32_t* counts = seg_counts + (int64_t)nseg * E1;
  int32_t* padded_off = counts + E1;
  const int ctas = nseg > 0 ? (nseg + PERM_WARPS - 1) / PERM_WARPS : 1;
  const size_t smem = (size_t)PERM_WARPS * E1 * 4;
  if (smem > 48 * 1024) return B200MOE_E_SHAPE;
  perm_count_kernel<<<ctas, PERM_WARPS * 32, smem, st>>>(topk_ids, numel, E1, nseg, seg_counts, sorted_token_ids,
                                                        sorted_token_ids ? sorted_cap : 0);
  int rc = check_launch();
  if (rc) return rc;
  perm_segscan_kernel<<<E1, 256, 0, st>>>(seg_counts, nseg, E1, counts);
  if ((rc = check_launch())) return rc;
  perm_experts_kernel<<<1, 1024, 0, st>>>(counts, E1, block, padded_off, expert_offsets, expert_ids,
                                          expert_ids ? expert_ids_cap : 0, num_tokens_post_pad);
  if ((rc = check_launch())) return rc;
  if (nseg > 0) {
    perm_scatter_kernel<<<ctas, PERM_WARPS * 32, smem, st>>>(topk_ids, numel, E1, nseg, seg_counts, padded_off,
                                                            expert_offsets, sorted_token_ids, sorted_routes, inv_routes);
    if ((rc = check_launch())) return rc;
  }
  return 0;
}
}  // namespace b200moe

extern "C" int b200moe_permute(const int32_t* topk_ids, int numel, int num_experts, int block, int32_t* sorted_token_ids,
                               int sorted_cap, int32_t* expert_ids, int expert_ids_cap, int32_t* num_tokens_post_pad,
                               int32_t* sorted_routes, int32_t* expert_offsets, void* workspace, int64_t workspace_bytes,
                               void* stream) {
  return b200moe::permute_with_inverse(topk_ids, numel, num_experts, block, sorted_token_ids, sorted_cap, expert_ids,
                                       expert_ids_cap, num_tokens_post_pad, sorted_routes, expert_offsets, nullptr, workspace,
                                       workspace_bytes, stream);
}
