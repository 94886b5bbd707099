// Expert-slot cache: slot tables, LRU ensure (device kernel + host twin), materialize, reset, miss fills.
#include <algorithm>
#include <vector>

#include "common.cuh"

namespace b200moe {

constexpr int LRU_THREADS = 1024;
constexpr int SLOT_BITS = 20;  // victim key = usage << SLOT_BITS | slot

__global__ void slot_reset_kernel(b200moe_slot_tables t) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int64_t total_ids = (int64_t)t.num_layers * t.num_experts;
  if (i < total_ids) t.slot_for_id[i] = -1;
  if (i < t.cache_size) {
    t.id_of_slot[i] = -1;
    t.usage[i] = 0;
  }
  if (i == 0) {
    *t.step = 0;
    *t.num_indices = 0;
  }
}

B200MOE_DEVICE unsigned long long block_min_u64(unsigned long long v, unsigned long long* scratch) {
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other < v ? other : v;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    unsigned long long w = lane < (blockDim.x >> 5) ? scratch[lane] : ~0ull;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const unsigned long long other = __shfl_xor_sync(0xffffffffu, w, o);
      w = other < w ? other : w;
    }
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  const unsigned long long r = scratch[32];
  __syncthreads();
  return r;
}

// One CTA.  E <= LRU_THREADS (one expert per thread), any S < 2^SLOT_BITS.
__global__ void __launch_bounds__(LRU_THREADS) slot_ensure_kernel(b200moe_slot_tables t, int layer,
                                                                  const int32_t* __restrict__ ids, int n_ids,
                                                                  int32_t* __restrict__ ids_out) {
  __shared__ int32_t active[LRU_THREADS];
  __shared__ int32_t miss_list[LRU_THREADS];
  __shared__ int32_t warp_cnt[2][32];
  __shared__ unsigned long long red[33];
  __shared__ int32_t totals[2];
  const int E = t.num_experts, S = t.cache_size;
  const int base = layer * E;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const long long step = *t.step + 1;

  active[tid] = 0;
  __syncthreads();
  for (int i = tid; i < n_ids; i += LRU_THREADS) {
    const int id = ids[i];
    if (id >= 0 && id < E) active[id] = 1;  // duplicates store the same value
  }
  __syncthreads();

  // hits bump, misses get their ascending-id rank
  int is_active = 0, is_miss = 0;
  if (tid < E && active[tid]) {
    is_active = 1;
    const int slot = t.slot_for_id[base + tid];
    if (slot >= 0) t.usage[slot] = step; else is_miss = 1;
  }
  const unsigned miss_ballot = __ballot_sync(0xffffffffu, is_miss);
  const unsigned act_ballot = __ballot_sync(0xffffffffu, is_active);
  if (lane == 0) {
    warp_cnt[0][warp] = __popc(miss_ballot);
    warp_cnt[1][warp] = __popc(act_ballot);
  }
  __syncthreads();
  int miss_before = 0;
  for (int w = 0; w < warp; ++w) miss_before += warp_cnt[0][w];
  if (is_miss) miss_list[miss_before + __popc(miss_ballot & ((1u << lane) - 1u))] = tid;
  if (tid == 0) {
    int m = 0, a = 0;
    for (int w = 0; w < 32; ++w) {
      m += warp_cnt[0][w];
      a += warp_cnt[1][w];
    }
    totals[0] = m;
    totals[1] = a;
  }
  __syncthreads();
  const int n_miss = totals[0];

  // victims: ascending (usage, slot) among slots with usage != step; a paired slot gets usage = step
  // and so drops out of the next round by itself.
  int paired = 0;
  for (int r = 0; r < n_miss; ++r) {
    unsigned long long best = ~0ull;
    for (int s = tid; s < S; s += LRU_THREADS) {
      const long long u = t.usage[s];
      if (u != step) {
        const unsigned long long key = ((unsigned long long)u << SLOT_BITS) | (unsigned)s;
        best = key < best ? key : best;
      }
    }
    best = block_min_u64(best, red);
    if (best == ~0ull) break;  // more misses than evictable slots: the rest stay unmapped
    if (tid == 0) {
      const int v = (int)(best & ((1u << SLOT_BITS) - 1u));
      const int e = miss_list[r];
      const int old = t.id_of_slot[v];
      if (old >= 0) t.slot_for_id[old] = -1;
      t.id_of_slot[v] = base + e;
      t.slot_for_id[base + e] = v;
      t.usage[v] = step;
      t.src_indices[r] = e;
      t.evict_slots[r] = v;
    }
    ++paired;
    __syncthreads();
  }

  if (tid == 0) {
    *t.step = step;
    *t.num_indices = paired;
    if (t.stats != nullptr) {
      t.stats[0] += totals[1];
      t.stats[1] += n_miss;
      t.stats[2] += 1;
    }
  }
  __syncthreads();
  for (int i = tid; i < n_ids; i += LRU_THREADS) {
    const int id = ids[i];
    ids_out[i] = (id >= 0 && id < E) ? t.slot_for_id[base + id] : id;
  }
}

__global__ void __launch_bounds__(1024) slot_materialize_kernel(b200moe_slot_tables t, int layer) {
  // single CTA; two passes separated by a barrier so unmapping never races with the new mapping
  const int E = t.num_experts, S = t.cache_size;
  const int base = layer * E;
  for (int s = threadIdx.x; s < S; s += blockDim.x) {
    const int old = t.id_of_slot[s];
    const bool same = old >= base && old < base + E;
    if (same) {
      t.id_of_slot[s] = -1;
      t.usage[s] = 0;
    } else if (s < E && old >= 0) {
      t.slot_for_id[old] = -1;
    }
  }
  __syncthreads();
  const long long step = *t.step + 1;
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    t.id_of_slot[e] = base + e;
    t.slot_for_id[base + e] = e;
    t.usage[e] = step;
    t.evict_slots[e] = e;
    t.src_indices[e] = e;
  }
  if (threadIdx.x == 0) {
    *t.step = step;
    *t.num_indices = E;
  }
}

// rows of 16-byte units; grid = blocks_per_bank * num_banks
__global__ void __launch_bounds__(1024) slot_gather_kernel(int num_banks, void* const* __restrict__ dst_banks,
                                                           const void* const* __restrict__ src_banks,
                                                           const int64_t* __restrict__ row_bytes,
                                                           const int32_t* __restrict__ evict_slots,
                                                           const int32_t* __restrict__ src_indices,
                                                           const int64_t* __restrict__ num_indices, int max_rows,
                                                           int blocks_per_bank) {
  const int bank = blockIdx.x / blocks_per_bank;
  const int part = blockIdx.x % blocks_per_bank;
  long long n = *num_indices;
  if (n > max_rows) n = max_rows;
  const int64_t units = row_bytes[bank] >> 4;
  char* dst = reinterpret_cast<char*>(dst_banks[bank]);
  const char* src = reinterpret_cast<const char*>(src_banks[bank]);
  for (long long i = 0; i < n; ++i) {
    const uint4* s = reinterpret_cast<const uint4*>(src + (int64_t)src_indices[i] * row_bytes[bank]);
    uint4* d = reinterpret_cast<uint4*>(dst + (int64_t)evict_slots[i] * row_bytes[bank]);
    for (int64_t u = (int64_t)part * blockDim.x + threadIdx.x; u < units; u += (int64_t)blocks_per_bank * blockDim.x)
      d[u] = s[u];
  }
}

static int check_tables(const b200moe_slot_tables* t, int layer) {
  if (!t || !t->slot_for_id || !t->id_of_slot || !t->usage || !t->step || !t->src_indices || !t->evict_slots ||
      !t->num_indices)
    return B200MOE_E_NULL;
  if (t->num_layers < 1 || t->num_experts < 1 || t->cache_size < 1 || t->cache_size >= (1 << SLOT_BITS) ||
      layer < 0 || layer >= t->num_layers)
    return B200MOE_E_SHAPE;
  return 0;
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_slot_reset(const b200moe_slot_tables* t, void* stream) {
  int rc = check_tables(t, 0);
  if (rc) return rc;
  const int64_t n = std::max<int64_t>((int64_t)t->num_layers * t->num_experts, t->cache_size);
  slot_reset_kernel<<<(unsigned)((n + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*t);
  return check_launch();
}

extern "C" int b200moe_slot_ensure(const b200moe_slot_tables* t, int layer, const int32_t* ids, int n_ids,
                                   int32_t* ids_out, void* stream) {
  int rc = check_tables(t, layer);
  if (rc) return rc;
  if (n_ids < 0 || t->num_experts > LRU_THREADS) return B200MOE_E_SHAPE;
  if (n_ids > 0 && (!ids || !ids_out)) return B200MOE_E_NULL;
  slot_ensure_kernel<<<1, LRU_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*t, layer, ids, n_ids, ids_out);
  return check_launch();
}

extern "C" int b200moe_slot_ensure_host(const b200moe_slot_tables* t, int layer, const int32_t* ids, int n_ids,
                                        int32_t* ids_out) {
  int rc = check_tables(t, layer);
  if (rc) return rc;
  if (n_ids < 0) return B200MOE_E_SHAPE;
  if (n_ids > 0 && (!ids || !ids_out)) return B200MOE_E_NULL;
  const int E = t->num_experts, S = t->cache_size, base = layer * E;
  const int64_t step = *t->step + 1;
  std::vector<char> active(E, 0);
  for (int i = 0; i < n_ids; ++i)
    if (ids[i] >= 0 && ids[i] < E) active[ids[i]] = 1;
  std::vector<int> miss;
  int n_active = 0;
  for (int e = 0; e < E; ++e) {
    if (!active[e]) continue;
    ++n_active;
    const int slot = t->slot_for_id[base + e];
    if (slot >= 0) t->usage[slot] = step; else miss.push_back(e);
  }
  int paired = 0;
  if (!miss.empty()) {
    std::vector<std::pair<int64_t, int>> cand;
    cand.reserve(S);
    for (int s = 0; s < S; ++s)
      if (t->usage[s] != step) cand.emplace_back(t->usage[s], s);
    const size_t take = std::min(cand.size(), miss.size());
    std::partial_sort(cand.begin(), cand.begin() + take, cand.end());
    for (size_t r = 0; r < take; ++r) {
      const int v = cand[r].second, e = miss[r];
      const int old = t->id_of_slot[v];
      if (old >= 0) t->slot_for_id[old] = -1;
      t->id_of_slot[v] = base + e;
      t->slot_for_id[base + e] = v;
      t->usage[v] = step;
      t->src_indices[r] = e;
      t->evict_slots[r] = v;
      ++paired;
    }
  }
  *t->step = step;
  *t->num_indices = paired;
  if (t->stats) {
    t->stats[0] += n_active;
    t->stats[1] += (int64_t)miss.size();
    t->stats[2] += 1;
  }
  for (int i = 0; i < n_ids; ++i) {
    const int id = ids[i];
    ids_out[i] = (id >= 0 && id < E) ? t->slot_for_id[base + id] : id;
  }
  return 0;
}

extern "C" int b200moe_slot_materialize(const b200moe_slot_tables* t, int layer, void* stream) {
  int rc = check_tables(t, layer);
  if (rc) return rc;
  if (t->cache_size < t->num_experts) return B200MOE_E_SHAPE;
  slot_materialize_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(*t, layer);
  return check_launch();
}

extern "C" int b200moe_slot_fill(int num_banks, void* const* dst_banks, const void* const* src_banks,
                                 const int64_t* row_bytes, const int32_t* evict_slots_host,
                                 const int32_t* src_indices_host, int n, void* stream) {
  if (n == 0) return 0;
  if (!dst_banks || !src_banks || !row_bytes || !evict_slots_host || !src_indices_host) return B200MOE_E_NULL;
  if (num_banks < 1 || n < 0) return B200MOE_E_SHAPE;
  for (int b = 0; b < num_banks; ++b)
    if (!dst_banks[b] || !src_banks[b] || row_bytes[b] <= 0) return B200MOE_E_NULL;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  for (int i = 0; i < n; ++i) {
    if (evict_slots_host[i] < 0 || src_indices_host[i] < 0) return B200MOE_E_SHAPE;
    for (int b = 0; b < num_banks; ++b) {
      char* d = reinterpret_cast<char*>(dst_banks[b]) + (int64_t)evict_slots_host[i] * row_bytes[b];
      const char* s = reinterpret_cast<const char*>(src_banks[b]) + (int64_t)src_indices_host[i] * row_bytes[b];
      cudaError_t e = cudaMemcpyAsync(d, s, (size_t)row_bytes[b], cudaMemcpyDefault, st);
      if (e != cudaSuccess) return (int)e;
    }
  }
  return 0;
}

extern "C" int b200moe_slot_gather(int num_banks, void* const* dst_banks_dev, const void* const* src_banks_dev,
                                   const int64_t* row_bytes_dev, const int32_t* evict_slots,
                                   const int32_t* src_indices, const int64_t* num_indices, int max_rows,
                                   int blocks_per_bank, void* stream) {
  if (!dst_banks_dev || !src_banks_dev || !row_bytes_dev || !evict_slots || !src_indices || !num_indices)
    return B200MOE_E_NULL;
  if (num_banks < 1 || max_rows < 0 || blocks_per_bank < 1) return B200MOE_E_SHAPE;
  slot_gather_kernel<<<num_banks * blocks_per_bank, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      num_banks, dst_banks_dev, src_banks_dev, row_bytes_dev, evict_slots, src_indices, num_indices, max_rows,
      blocks_per_bank);
  return check_launch();
}

// ------------------------------------------------------------------------------------------------
// One-layer-ahead speculative prefetch (pre-gate): which experts will the NEXT layer's router pick, judged
// from the residual stream that leaves this layer?  (freetoken/python/freetoken/moe/pregate.py:77-117)
//   logits[e] = sum_h gate_w[e, h] * bf16(residual[h] * rsqrt(mean(residual^2) + eps) * norm_w[h])     (fp32)
//   query[0 .. width) = the first `cap` of the top_k predictions (score order, ties: lower id; NaN ranks last)
//   whose slot is unmapped, padded with the first of them -- or with the top-1 prediction when none misses.
// The query then goes through the unchanged LRU ensure; a wrong prediction costs bus traffic and residency only.
// ------------------------------------------------------------------------------------------------
namespace b200moe {

// grid = E / 8, block = 256: warp w of a block -> expert 8 * blockIdx.x + w
__global__ void __launch_bounds__(256) pregate_logits_kernel(const __nv_bfloat16* __restrict__ residual,
                                                             const __nv_bfloat16* __restrict__ norm_w,
                                                             const __nv_bfloat16* __restrict__ gate_w, int64_t gate_stride,
                                                             float* __restrict__ logits, float eps, int H, int E) {
  __shared__ float red[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float ss = 0.f;
  for (int h = tid; h < H; h += 256) {
    const float v = __bfloat162float(residual[h]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if (lane == 0) red[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) tot += red[w];
  const float inv = 1.0f / sqrtf(tot / (float)H + eps);
  const int e = blockIdx.x * 8 + warp;
  if (e >= E) return;
  const __nv_bfloat16* g = gate_w + (int64_t)e * gate_stride;
  float acc = 0.f;
  for (int h = lane; h < H; h += 32) {
    const float y = bf16_round(__bfloat162float(residual[h]) * inv * __bfloat162float(norm_w[h]));
    acc += __bfloat162float(g[h]) * y;
  }
  acc = warp_sum(acc);
  if (lane == 0) logits[e] = acc;
}

// one warp; E <= 512
__global__ void __launch_bounds__(32) pregate_select_kernel(const float* __restrict__ logits, const int32_t* __restrict__ slot_row,
                                                            int32_t* __restrict__ query, int cap, int E, int top_k, int width) {
  const int lane = threadIdx.x;
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int n = i * 32 + lane;
    float x = n < E ? logits[n] : -INFINITY;
    if (!(x == x)) x = -INFINITY;
    v[i] = x;
  }
  int count = 0, first = 0, top1 = 0;
  for (int k = 0; k < top_k; ++k) {
    // highest value, lowest id among equals (an all -inf tail therefore repeats the lowest id, as the reference does)
    float best = -INFINITY;
    int arg = 1 << 30;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int n = i * 32 + lane;
      if (n < E && (v[i] > best || (v[i] == best && n < arg))) {
        best = v[i];
        arg = n;
      }
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) {
        best = ob;
        arg = oa;
      }
    }
    const int win = min(arg, E - 1);
    if (k == 0) top1 = win;
    const bool miss = slot_row[win] < 0 && count < cap;
    if (miss) {
      if (lane == 0) query[count] = win;
      if (count == 0) first = win;
      ++count;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (i * 32 + lane == win) v[i] = -INFINITY;
  }
  const int pad = count > 0 ? first : top1;
  for (int p = count + lane; p < width; p += 32) query[p] = pad;
}

}  // namespace b200moe

extern "C" int b200moe_pregate_predict(const void* residual, const void* norm_w, float eps, const void* gate_w,
                                       int64_t gate_stride, int hidden, int num_experts, const int32_t* slot_row, int cap,
                                       int top_k, float* logits, int32_t* query, int width, void* stream) {
  if (!residual || !norm_w || !gate_w || !slot_row || !logits || !query) return B200MOE_E_NULL;
  if (hidden < 1 || num_experts < 8 || num_experts % 8 || num_experts > 512 || top_k < 1 || top_k > num_experts || cap < 0 ||
      width < 1 || cap > width)
    return B200MOE_E_SHAPE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  b200moe::pregate_logits_kernel<<<num_experts / 8, 256, 0, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(residual), reinterpret_cast<const __nv_bfloat16*>(norm_w),
      reinterpret_cast<const __nv_bfloat16*>(gate_w), gate_stride, logits, eps, hidden, num_experts);
  int rc = b200moe::check_launch();
  if (rc) return rc;
  b200moe::pregate_select_kernel<<<1, 32, 0, st>>>(logits, slot_row, query, cap, num_experts, top_k, width);
  return b200moe::check_launch();
}

// ------------------------------------------------------------------------------------------------
// Prefill through the cache, selected-experts form: which of the experts a chunk routes to are resident
// (slot >= first_lru_slot: outside the two prefill buffers) and which must come from the host bank?
// (freetoken/python/freetoken/moe/offload_cache.py:1160-1200 with offload_kernels.py:63-113: mark_selected +
// prefill_split_compact.)  Both lists are in ascending expert id; destination rows are buffer rows
// buffer_row0 + expert (position == expert id inside a buffer).  Reads the slot map only: no usage, no stats.
// ------------------------------------------------------------------------------------------------
namespace b200moe {

__global__ void __launch_bounds__(1024) prefill_split_kernel(const int32_t* __restrict__ topk_ids, int n_ids,
                                                             const int32_t* __restrict__ slot_row, int E, int first_lru_slot,
                                                             int buffer_row0, int select_all, int32_t* __restrict__ hit_dst,
                                                             int32_t* __restrict__ hit_src, int32_t* __restrict__ miss_dst,
                                                             int32_t* __restrict__ miss_src, int64_t* __restrict__ counts) {
  __shared__ int selected[1024];
  __shared__ int whit[32], wmiss[32];
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  selected[e] = select_all;
  __syncthreads();
  if (!select_all)
    for (int i = e; i < n_ids; i += 1024) {
      const int id = topk_ids[i];
      if (id >= 0 && id < E) selected[id] = 1;
    }
  __syncthreads();
  const bool sel = e < E && selected[e];
  const int slot = e < E ? slot_row[e] : -1;
  const bool hit = sel && slot >= first_lru_slot, miss = sel && !hit;
  const unsigned hb = __ballot_sync(0xffffffffu, hit), mb = __ballot_sync(0xffffffffu, miss);
  if (lane == 0) {
    whit[warp] = __popc(hb);
    wmiss[warp] = __popc(mb);
  }
  __syncthreads();
  int hbase = 0, mbase = 0, htot = 0, mtot = 0;
  for (int w = 0; w < 32; ++w) {
    if (w < warp) {
      hbase += whit[w];
      mbase += wmiss[w];
    }
    htot += whit[w];
    mtot += wmiss[w];
  }
  const unsigned below = (1u << lane) - 1u;
  if (hit) {
    const int i = hbase + __popc(hb & below);
    hit_dst[i] = buffer_row0 + e;
    hit_src[i] = slot;
  }
  if (miss) {
    const int i = mbase + __popc(mb & below);
    miss_dst[i] = buffer_row0 + e;
    miss_src[i] = e;
  }
  if (e == 0) {
    counts[0] = htot;
    counts[1] = mtot;
  }
}

}  // namespace b200moe

extern "C" int b200moe_prefill_split(const int32_t* topk_ids, int n_ids, const int32_t* slot_row, int num_experts,
                                     int first_lru_slot, int buffer_row0, int select_all, int32_t* hit_dst, int32_t* hit_src,
                                     int32_t* miss_dst, int32_t* miss_src, int64_t* counts, void* stream) {
  if (!slot_row || !hit_dst || !hit_src || !miss_dst || !miss_src || !counts) return B200MOE_E_NULL;
  if (!select_all && (!topk_ids || n_ids < 0)) return B200MOE_E_NULL;
  if (num_experts < 1 || num_experts > 1024) return B200MOE_E_SHAPE;
  b200moe::prefill_split_kernel<<<1, 1024, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      topk_ids, n_ids, slot_row, num_experts, first_lru_slot, buffer_row0, select_all, hit_dst, hit_src, miss_dst, miss_src,
      counts);
  return b200moe::check_launch();
}
