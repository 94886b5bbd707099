// Router selection shared by the stand-alone router kernel and the decode kernels that route in their prologue.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace b200moe {

// One warp, one token: fp32 softmax over E logits (lane j owns experts j, j+32, ...), then top_k rounds of
// (highest logit, lowest id among equals); NaN logits rank as -1e30.  Writes the selected probabilities
// (renormalised if asked) and ids, in selection order, to w_out / id_out (global or shared memory).
// WEIGHTS = false: only the ids (no softmax; w_out is not touched and may be null) -- what a consumer that needs the
// experts first and their weights later runs on its critical path.
template <int NPL, typename LogitT, bool WEIGHTS = true>
B200MOE_DEVICE void router_select(const LogitT* __restrict__ src, int E, int top_k, int renormalize, int lane,
                                  float* w_out, int32_t* id_out) {
  float raw[NPL], prob[NPL], cur[NPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    raw[i] = e < E ? (float)src[e] : -INFINITY;
    mx = fmaxf(mx, raw[i]);  // fmaxf ignores NaN, as the reference's max reduction does
    prob[i] = 0.f;
  }
  if constexpr (WEIGHTS) {
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      prob[i] = e < E ? expf(raw[i] - mx) : 0.f;
      sum += prob[i];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int i = 0; i < NPL; ++i) prob[i] = prob[i] / sum;
  }
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    cur[i] = e < E ? (raw[i] == raw[i] ? raw[i] : -1e30f) : -INFINITY;
  }
  float my_w = 0.f;  // lane k keeps the k-th selection of the current group of 32
  int my_id = 0;
  float wsum = 0.f;
  // bf16 logits: (value, id) fits one 32-bit key whose integer order is the selection order -- value rank in the
  // high bits (twice the order-preserving code of the bf16 bits; NaN takes the odd rank between the two bf16 values
  // around -1e30), 511 - id below it (lowest id wins among equals); a round is a few integer max and one warp
  // reduction instead of compare-and-select chains on (float, int) pairs.  Keys of taken or absent experts are 0.
  constexpr bool KEYED = std::is_same<LogitT, __nv_bfloat16>::value && NPL <= 16;
  uint32_t key[NPL];
  if constexpr (KEYED) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      uint32_t b = e < E ? (uint32_t)__bfloat16_as_ushort(src[e]) : 0xff80u;
      const bool nan = (b & 0x7fffu) > 0x7f80u;
      const uint32_t ord = (b & 0x8000u) ? (~b & 0xffffu) : (b | 0x8000u);
      const uint32_t rank = nan ? 2u * 0x0eb5u + 1u : 2u * ord;  // 0x0eb5: code of 0xf14a, the bf16 just below -1e30
      key[i] = e < E ? (rank << 9) | (uint32_t)(511 - e) : 0u;
    }
  }
  for (int k = 0; k < top_k; ++k) {
    int bi;
    if constexpr (KEYED) {
      uint32_t best = key[0];
#pragma unroll
      for (int i = 1; i < NPL; ++i) best = max(best, key[i]);
      best = __reduce_max_sync(0xffffffffu, best);
      bi = 511 - (int)(best & 511u);
    } else {
      float bv = cur[0];
      bi = lane;
#pragma unroll
      for (int i = 1; i < NPL; ++i) {
        if (cur[i] > bv) {  // strict: the first (lowest id) of equal values stays
          bv = cur[i];
          bi = lane + 32 * i;
        }
      }
#pragma unroll
      for (int o = 16; o; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
          bv = ov;
          bi = oi;
        }
      }
    }
    float p = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      if (lane + 32 * i == bi) {
        p = prob[i];
        cur[i] = -INFINITY;
        key[i] = 0u;
      }
    }
    p = __shfl_sync(0xffffffffu, p, bi & 31);
    wsum += p;
    if (lane == (k & 31)) {
      my_w = p;
      my_id = bi;
    }
    if ((k & 31) == 31 || k == top_k - 1) {  // flush a group of up to 32 selections
      const int kk = (k & ~31) + lane;
      if (kk <= k) {
        if constexpr (WEIGHTS) w_out[kk] = my_w;
        id_out[kk] = my_id;
      }
    }
  }
  __syncwarp();
  if (WEIGHTS && renormalize) {
    const float d = wsum > 0.f ? wsum : 1.f;
    for (int kk = lane; kk < top_k; kk += 32) w_out[kk] = w_out[kk] / d;  // each lane re-reads what it wrote
  }
  __syncwarp();
}

// The weights of experts that are already selected (ids[0..top_k) in selection order, shared or global memory): the
// same arithmetic as router_select -- softmax over all E logits, the selected probabilities, their sum in selection
// order, the renormalising division -- without the selection rounds.  One warp; writes w_out[0..top_k), top_k <= 32.
template <int NPL, typename LogitT>
B200MOE_DEVICE void router_weights(const LogitT* __restrict__ src, int E, int top_k, int renormalize, int lane,
                                   const int32_t* ids, float* w_out) {
  float raw[NPL];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    raw[i] = e < E ? (float)src[e] : -INFINITY;
    mx = fmaxf(mx, raw[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    sum += e < E ? expf(raw[i] - mx) : 0.f;
  }
  sum = warp_sum(sum);
  float p = 0.f;
  if (lane < top_k) p = expf((float)src[ids[lane]] - mx) / sum;
  float wsum = 0.f;
  for (int k = 0; k < top_k; ++k) wsum += __shfl_sync(0xffffffffu, p, k);
  if (renormalize) p = p / (wsum > 0.f ? wsum : 1.f);
  if (lane < top_k) w_out[lane] = p;
}

}  // namespace b200moe
