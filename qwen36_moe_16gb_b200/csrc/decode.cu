// Decode path (1..8 tokens): HBM-bound GEMVs that stream the FP4 expert rows with 128-bit loads.
//
// Every warp owns a 16-row x K-slice tile of one weight matrix.  Lane (g = lane/4, t = lane%4) loads
// 64 contiguous bytes of row g and of row g+8; the four lanes of a group cover 256 contiguous bytes
// of a row.  The multiply-accumulate runs on the warp MMA (m16n8k16, fp32 accumulate) with the weight
// fragment built IN REGISTERS from the packed codes (cvt e2m1x2 -> f16x2, times the e4m3 block scale,
// both exact), so the only per-element ALU work is the unpack.  The activation row is staged once per
// CTA in shared memory as fp16 scaled by a power of two (exact for bf16 inputs unless an element is
// more than 2^28 below the row maximum).  Because any permutation of k applied to both operands leaves
// a dot product unchanged, fragments take k in load order and no shuffle is needed.
#include <algorithm>
#include <mutex>
#include <utility>
#include <vector>

#include "common.cuh"
#include "router.cuh"

namespace b200moe {

constexpr int FP4_SLICE = 512;   // k per warp pass: 4 lanes x 128

__host__ __device__ __forceinline__ int xs_idx128(int k) { return k + ((k >> 7) << 3); }  // 16 B pad per 128 halves
__host__ __device__ __forceinline__ int xs_idx32(int k) { return k + ((k >> 5) << 3); }   // 16 B pad per 32 halves

struct Fp4Regs {
  uint4 qa[4], qb[4];
  uint2 sa, sb;
};

// pa/pb: row start of this lane's two rows (packed bytes); sa/sb: their scale rows; k0: slice start.
B200MOE_DEVICE void fp4_issue_loads(Fp4Regs& r, const uint8_t* pa, const uint8_t* pb, const uint8_t* sa,
                                    const uint8_t* sb, int k0, int t) {
  const int byte0 = (k0 >> 1) + 64 * t;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    r.qa[c] = ldg_nc_keep_v4(pa + byte0 + 16 * c);
    r.qb[c] = ldg_nc_keep_v4(pb + byte0 + 16 * c);
  }
  r.sa = ldg_nc_v2(sa + (k0 >> 4) + 8 * t);
  r.sb = ldg_nc_v2(sb + (k0 >> 4) + 8 * t);
}

// xs: fp16 activation row in shared memory (xs_idx128 layout).
// acc: four independent accumulator chains (consecutive MMAs never wait on each other); sum them with acc_sum.
B200MOE_DEVICE void fp4_compute(const Fp4Regs& r, const __half* xs, int k0, int t, float (&acc)[4][4]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint32_t ra = (c < 2 ? r.sa.x : r.sa.y) >> (16 * (c & 1));
    const uint32_t rb = (c < 2 ? r.sb.x : r.sb.y) >> (16 * (c & 1));
    const uint32_t s2a = e4m3x2_to_f16x2(ra & 0xffffu);  // {block 2c, block 2c+1}
    const uint32_t s2b = e4m3x2_to_f16x2(rb & 0xffffu);
    const uint32_t wa[4] = {r.qa[c].x, r.qa[c].y, r.qa[c].z, r.qa[c].w};
    const uint32_t wb[4] = {r.qb[c].x, r.qb[c].y, r.qb[c].z, r.qb[c].w};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const uint32_t sA = w < 2 ? dup_lo16(s2a) : dup_hi16(s2a);
      const uint32_t sB = w < 2 ? dup_lo16(s2b) : dup_hi16(s2b);
      uint32_t ha[4], hb[4];
      e2m1x8_to_f16x2(wa[w], ha);
      e2m1x8_to_f16x2(wb[w], hb);
      const int k = k0 + 128 * t + 32 * c + 8 * w;
      const uint4 xv = *reinterpret_cast<const uint4*>(xs + xs_idx128(k));
      uint32_t a[4];
      a[0] = hmul2_u32(ha[0], sA); a[1] = hmul2_u32(hb[0], sB);
      a[2] = hmul2_u32(ha[1], sA); a[3] = hmul2_u32(hb[1], sB);
      mma_f16_16816(acc[(2 * w) & 3], a, xv.x, xv.y);
      a[0] = hmul2_u32(ha[2], sA); a[1] = hmul2_u32(hb[2], sB);
      a[2] = hmul2_u32(ha[3], sA); a[3] = hmul2_u32(hb[3], sB);
      mma_f16_16816(acc[(2 * w + 1) & 3], a, xv.z, xv.w);
    }
  }
}

B200MOE_DEVICE void acc_zero(float (&acc)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
}
// element j of the summed fragment (0: row g col 2t, 2: row g+8 col 2t)
B200MOE_DEVICE float acc_sum(const float (&acc)[4][4], int j) { return (acc[0][j] + acc[1][j]) + (acc[2][j] + acc[3][j]); }

// Stage one bf16 row of n values (n % 8 == 0) as scaled fp16 into xs (xs_idx128 layout) with `nthr`
// cooperating threads (a whole CTA with red != nullptr, or one warp with red == nullptr).
// Returns the inverse of the power-of-two scale.
B200MOE_DEVICE float stage_row_f16(const __nv_bfloat16* __restrict__ row, int n, __half* xs, int tid, int nthr,
                                   float* red) {
  constexpr int KEEP = 4;  // 16-byte pieces a thread keeps in registers between the two phases
  const bool fits = n <= nthr * 8 * KEEP;
  uint4 held[KEEP];
  float amax = 0.f;
#pragma unroll
  for (int p = 0; p < KEEP; ++p) {
    const int i = (tid + p * nthr) * 8;
    held[p] = make_uint4(0, 0, 0, 0);
    if (i < n) held[p] = *reinterpret_cast<const uint4*>(row + i);
    const uint32_t w[4] = {held[p].x, held[p].y, held[p].z, held[p].w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      amax = fmaxf(amax, fabsf(bf16_bits_to_float(w[j] & 0xffffu)));
      amax = fmaxf(amax, fabsf(__uint_as_float(w[j] & 0xffff0000u)));
    }
  }
  if (!fits) {
    for (int i = (tid + KEEP * nthr) * 8; i < n; i += nthr * 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(row + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        amax = fmaxf(amax, fabsf(bf16_bits_to_float(w[j] & 0xffffu)));
        amax = fmaxf(amax, fabsf(__uint_as_float(w[j] & 0xffff0000u)));
      }
    }
  }
  amax = warp_max(amax);
  if (red != nullptr) {
    if ((tid & 31) == 0) red[tid >> 5] = amax;
    __syncthreads();
    amax = 0.f;
    for (int w = 0; w < (nthr >> 5); ++w) amax = fmaxf(amax, red[w]);
  }
  float scale, inv;
  f16_row_scale(amax, scale, inv);
  auto put = [&](int i, const uint4& v) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 h = __floats2half2_rn(bf16_bits_to_float(w[j] & 0xffffu) * scale,
                                          __uint_as_float(w[j] & 0xffff0000u) * scale);
      o[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(xs + xs_idx128(i)) = make_uint4(o[0], o[1], o[2], o[3]);
  };
#pragma unroll
  for (int p = 0; p < KEEP; ++p) {
    const int i = (tid + p * nthr) * 8;
    if (i < n) put(i, held[p]);
  }
  if (!fits)
    for (int i = (tid + KEEP * nthr) * 8; i < n; i += nthr * 8) put(i, *reinterpret_cast<const uint4*>(row + i));
  return inv;
}

// Programmatic dependent launch: every kernel lets its successor start early (launch_dependents) and blocks
// (wait) before it touches anything a predecessor wrote.  Weight loads that depend on nothing are issued
// before the wait, so they stream from HBM while the predecessor is still running.  Without the launch
// attribute both instructions do nothing.
B200MOE_DEVICE void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
B200MOE_DEVICE void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ------------------------------------------------------------------------------------------------
// GEMM1 + SwiGLU.  grid = (I / (8*TILES), routes [+1 for the shared expert's activation]).
// A row tile pairs gate rows n..n+7 (fragment rows 0..7) with up rows I+n..I+n+7 (fragment rows 8..15),
// so a lane ends up holding gate and up of the same output and applies SwiGLU in registers.
// KS warps share a tile along K (KS=4: every warp makes one pass, lowest latency; KS=1: one warp walks
// all of K with the next pass's loads in flight while it computes, highest throughput).
// When `ids` is null the CTA routes its own token first (top-k of the token's logits, redundantly per
// CTA) and CTA (0, first route of the token) publishes weights and ids for the second GEMM.
// ------------------------------------------------------------------------------------------------
constexpr int G1_WARPS = 8;

template <int KS>
B200MOE_DEVICE void decode_gemm1_body(unsigned char* smem_raw, int bx, int r, const __nv_bfloat16* __restrict__ x,
                                      const b200moe_banks& bk, const int32_t* __restrict__ ids, bool ids_settled,
                                      const __nv_bfloat16* __restrict__ logits, int E, float* __restrict__ topk_w_out,
                                      int32_t* __restrict__ topk_ids_out, int top_k, int NT,
                                      __nv_bfloat16* __restrict__ ic2) {
  // NT = row tiles of this CTA; warp = (tile slot, K share); a warp walks its (tile, pass) items with the next
  // item's loads in flight while it multiplies the current one.
  const int H = bk.hidden, I = bk.intermediate;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  __half* xs = reinterpret_cast<__half*>(smem_raw);
  float* red = reinterpret_cast<float*>(smem_raw + (size_t)xs_idx128(H) * 2);  // [32]
  float* sel_w = red + 32;                                                     // [8]
  int32_t* sel_id = reinterpret_cast<int32_t*>(sel_w + 8);                     // [8]
  float* part = sel_w + 16;                                                    // [NT][KS][16]

  const int token = r / top_k, kk = r - token * top_k;
  int slot;
  float inv = 1.f;
  if (ids != nullptr) {
    // `ids_settled`: the ids were written before the first kernel of this launch sequence started (the host-planned
    // offload step copies them in ahead of the layer loop).  Otherwise the previous kernel in the stream may have
    // produced them (router top-k, slot-cache ensure), and its writes are only visible after the dependency wait.
    if (!ids_settled) pdl_wait();
    slot = ids[r];
  } else {
    // Resident block: the previous kernel is the dense rows, which produce the logits but not x, and which raise
    // their launch trigger only after their own dependency wait -- so x is complete when this kernel starts and can
    // be staged before the wait, while the dense rows are still running.
    inv = stage_row_f16(x + (int64_t)token * H, H, xs, tid, blockDim.x, red);
    pdl_wait();  // the logits come from the previous kernel
    if (warp == 0) {  // the experts only: this kernel does not use the router weights
      const __nv_bfloat16* row = logits + (int64_t)token * E;
      if (E <= 256) router_select<8, __nv_bfloat16, false>(row, E, top_k, 1, lane, nullptr, sel_id);
      else router_select<16, __nv_bfloat16, false>(row, E, top_k, 1, lane, nullptr, sel_id);
    }
    __syncthreads();  // also: every thread's part of xs is in shared memory
    slot = sel_id[kk];
  }
  constexpr int TS = G1_WARPS / KS;  // tile slots
  const int tslot = warp / KS, ks = warp % KS;
  const int g = lane >> 2, t = lane & 3;
  const bool live = slot >= 0 && slot < bk.num_slots;
  const int passes = (H / FP4_SLICE + KS - 1 - ks) / KS;          // passes of this warp per tile
  const int my_tiles = NT > tslot ? (NT - tslot + TS - 1) / TS : 0;
  const int items = live ? my_tiles * passes : 0;
  const uint8_t* pbase = bk.gate_up + (int64_t)(live ? slot : 0) * bk.slot_stride[0];
  const uint8_t* sbase = bk.gate_up_scale + (int64_t)(live ? slot : 0) * bk.slot_stride[1];
  auto row_of = [&](int it) { return (bx * NT + tslot + (it / passes) * TS) * 8 + g; };  // gate row
  auto k_of = [&](int it) { return (ks + (it % passes) * KS) * FP4_SLICE; };
  auto issue = [&](Fp4Regs& rg, int it) {
    const int n = row_of(it);
    fp4_issue_loads(rg, pbase + (int64_t)n * (H >> 1), pbase + (int64_t)(I + n) * (H >> 1),
                    sbase + (int64_t)n * (H >> 4), sbase + (int64_t)(I + n) * (H >> 4), k_of(it), t);
  };
  Fp4Regs ra, rb;
  if (items > 0) issue(ra, 0);  // weights: in flight across the dependency wait and while x is staged
  if (ids != nullptr) {
    pdl_wait();
    inv = stage_row_f16(x + (int64_t)token * H, H, xs, tid, blockDim.x, red);
    __syncthreads();
  } else if (bx == 0 && kk == 0 && warp == 0) {
    // one CTA per token publishes weights and ids for the second GEMM; the softmax runs here, while this warp's
    // weight rows are on their way
    const __nv_bfloat16* row = logits + (int64_t)token * E;
    if (E <= 256) router_weights<8, __nv_bfloat16>(row, E, top_k, 1, lane, sel_id, sel_w);
    else router_weights<16, __nv_bfloat16>(row, E, top_k, 1, lane, sel_id, sel_w);
    __syncwarp();
    if (lane < top_k) {
      topk_w_out[token * top_k + lane] = sel_w[lane];
      topk_ids_out[token * top_k + lane] = sel_id[lane];
    }
  }

  float acc[4][4];
  acc_zero(acc);
  const float* gl = bk.gate_up_global + (int64_t)(live ? slot : 0) * (bk.slot_stride[2] >> 2);
  auto finish = [&](int it) {
    if ((it % passes) != passes - 1) return;
    if (t == 0) {
      const int tile = tslot + (it / passes) * TS;
      const float gate = acc_sum(acc, 0), up = acc_sum(acc, 2);
      if (KS == 1) {
        const int n = row_of(it);
        const float g1 = bf16_round((gate * inv) * gl[n]);
        const float u1 = bf16_round((up * inv) * gl[I + n]);
        ic2[(int64_t)r * I + n] = __float2bfloat16_rn(silu_mul(g1, u1));
      } else {
        part[(tile * KS + ks) * 16 + g] = gate;
        part[(tile * KS + ks) * 16 + 8 + g] = up;
      }
    }
    acc_zero(acc);
  };
  for (int it = 0; it < items; it += 2) {
    if (it + 1 < items) issue(rb, it + 1);
    fp4_compute(ra, xs, k_of(it), t, acc);
    finish(it);
    if (it + 1 < items) {
      if (it + 2 < items) issue(ra, it + 2);
      fp4_compute(rb, xs, k_of(it + 1), t, acc);
      finish(it + 1);
    }
  }
  if (KS > 1 || !live) {
    __syncthreads();
    for (int o = tid; o < NT * 8; o += blockDim.x) {
      const int tile = o >> 3, gg = o & 7;
      const int n = (bx * NT + tile) * 8 + gg;
      float y = 0.f;
      if (live) {
        float gate = 0.f, up = 0.f;
#pragma unroll
        for (int s = 0; s < KS; ++s) {
          gate += part[(tile * KS + s) * 16 + gg];
          up += part[(tile * KS + s) * 16 + 8 + gg];
        }
        const float g1 = bf16_round((gate * inv) * gl[n]);
        const float u1 = bf16_round((up * inv) * gl[I + n]);
        y = silu_mul(g1, u1);
      }
      ic2[(int64_t)r * I + n] = __float2bfloat16_rn(y);
    }
  }
}

template <int KS>
__global__ void __launch_bounds__(G1_WARPS * 32, 2) decode_gemm1_kernel(
    const __nv_bfloat16* __restrict__ x, b200moe_banks bk, const int32_t* __restrict__ ids,
    const __nv_bfloat16* __restrict__ logits, int E, float* __restrict__ topk_w_out, int32_t* __restrict__ topk_ids_out,
    int top_k, int NT, __nv_bfloat16* __restrict__ ic2) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_launch_dependents();
  decode_gemm1_body<KS>(smem_raw, blockIdx.x, blockIdx.y, x, bk, ids, false, logits, E, topk_w_out, topk_ids_out, top_k, NT,
                        ic2);
}

// ------------------------------------------------------------------------------------------------
// GEMM2 * router weight, sum over the token's routes, optional shared expert + merge.
// grid = (H / (16*TPW), M).  Warp k < top_k: route k of the token, TPW row tiles of `down` one after the
// other (next tile's loads in flight while the current one is multiplied), K = I.
// Warps top_k .. top_k+3 (with_shared): K-quarters of the shared expert's bf16 `down` rows; their first
// loads do not depend on the previous kernel and are issued before the dependency wait.
// ------------------------------------------------------------------------------------------------
constexpr int SH_WARPS = 4;

struct BfRegs {
  uint4 qa[4], qb[4];
};
B200MOE_DEVICE void bf_issue(BfRegs& r, const __nv_bfloat16* wa, const __nv_bfloat16* wb, int k0, int t) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    r.qa[c] = ldg_nc_keep_v4(wa + k0 + 32 * t + 8 * c);
    r.qb[c] = ldg_nc_keep_v4(wb + k0 + 32 * t + 8 * c);
  }
}
// xs: bf16 activations in shared memory, xs_idx32 layout
B200MOE_DEVICE void bf_compute(const BfRegs& r, const __nv_bfloat16* xs, int k0, int t, float (&acc)[4][4]) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const uint4 xv = *reinterpret_cast<const uint4*>(xs + xs_idx32(k0 + 32 * t + 8 * c));
    uint32_t a[4] = {r.qa[c].x, r.qb[c].x, r.qa[c].y, r.qb[c].y};
    mma_bf16_16816(acc[(2 * c) & 3], a, xv.x, xv.y);
    uint32_t b[4] = {r.qa[c].z, r.qb[c].z, r.qa[c].w, r.qb[c].w};
    mma_bf16_16816(acc[(2 * c + 1) & 3], b, xv.z, xv.w);
  }
}

__global__ void __launch_bounds__(384) decode_gemm2_kernel(int TPW, const __nv_bfloat16* __restrict__ ic2, b200moe_banks bk,
                                                           const float* __restrict__ topk_w,
                                                           const int32_t* __restrict__ ids, int top_k,
                                                           const __nv_bfloat16* __restrict__ hs,
                                                           const __nv_bfloat16* __restrict__ shared_down, int SI,
                                                           const __nv_bfloat16* __restrict__ gate_logit,
                                                           __nv_bfloat16* __restrict__ out, int with_shared) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = bk.hidden, I = bk.intermediate;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int m = blockIdx.y, n0 = blockIdx.x * 16 * TPW;
  const int xs_stride = xs_idx128(I);                      // halves per route row
  __half* xs_all = reinterpret_cast<__half*>(smem_raw);    // [top_k][xs_stride]
  __nv_bfloat16* as = reinterpret_cast<__nv_bfloat16*>(smem_raw + (size_t)top_k * xs_stride * 2);  // [xs_idx32(SI)]
  float* ic3 = reinterpret_cast<float*>(smem_raw + (size_t)top_k * xs_stride * 2 + (size_t)xs_idx32(SI) * 2);  // [TPW][top_k][16]
  float* sh_part = ic3 + TPW * top_k * 16;                 // [TPW][SH_WARPS][16]
  pdl_launch_dependents();

  if (warp < top_k) {
    pdl_wait();
    const int r = m * top_k + warp;
    const int slot = ids[r];
    const bool live = slot >= 0 && slot < bk.num_slots;
    const int passes = I / FP4_SLICE, items = TPW * passes;
    if (live) {
      const uint8_t* pbase = bk.down + (int64_t)slot * bk.slot_stride[3];
      const uint8_t* sbase = bk.down_scale + (int64_t)slot * bk.slot_stride[4];
      const float* gl = bk.down_global + (int64_t)slot * (bk.slot_stride[5] >> 2);
      const float w = topk_w[r];
      auto issue = [&](Fp4Regs& rg, int it) {
        const int row = n0 + (it / passes) * 16 + g;
        fp4_issue_loads(rg, pbase + (int64_t)row * (I >> 1), pbase + (int64_t)(row + 8) * (I >> 1),
                        sbase + (int64_t)row * (I >> 4), sbase + (int64_t)(row + 8) * (I >> 4), (it % passes) * FP4_SLICE, t);
      };
      Fp4Regs ra, rb;
      issue(ra, 0);
      __half* xs = xs_all + warp * xs_stride;
      const float inv = stage_row_f16(ic2 + (int64_t)r * I, I, xs, lane, 32, nullptr);
      __syncwarp();
      float acc[4][4];
      acc_zero(acc);
      auto finish = [&](int it) {  // after the last pass of a tile: scale, weight, round, park in smem
        if ((it % passes) == passes - 1) {
          const int tile = it / passes;
          if (t == 0) {
            const int row = n0 + tile * 16 + g;
            ic3[(tile * top_k + warp) * 16 + g] = bf16_round(((acc_sum(acc, 0) * inv) * gl[row]) * w);
            ic3[(tile * top_k + warp) * 16 + 8 + g] = bf16_round(((acc_sum(acc, 2) * inv) * gl[row + 8]) * w);
          }
          acc_zero(acc);
        }
      };
      for (int it = 0; it < items; it += 2) {
        if (it + 1 < items) issue(rb, it + 1);
        fp4_compute(ra, xs, (it % passes) * FP4_SLICE, t, acc);
        finish(it);
        if (it + 1 < items) {
          if (it + 2 < items) issue(ra, it + 2);
          fp4_compute(rb, xs, ((it + 1) % passes) * FP4_SLICE, t, acc);
          finish(it + 1);
        }
      }
    } else if (t == 0) {
      for (int tile = 0; tile < TPW; ++tile) {
        ic3[(tile * top_k + warp) * 16 + g] = 0.f;
        ic3[(tile * top_k + warp) * 16 + 8 + g] = 0.f;
      }
    }
  } else if (with_shared) {
    const int j = warp - top_k;  // K quarter
    const int kpass = (SI + SH_WARPS * 128 - 1) / (SH_WARPS * 128);  // passes per tile for this warp
    const int items = TPW * kpass;
    auto issue = [&](BfRegs& rg, int it) {
      const int row = n0 + (it / kpass) * 16 + g;
      const int k0 = j * 128 + (it % kpass) * SH_WARPS * 128;
      if (k0 < SI) bf_issue(rg, shared_down + (int64_t)row * SI, shared_down + (int64_t)(row + 8) * SI, k0, t);
    };
    BfRegs ra, rb;
    issue(ra, 0);           // weights only: legal before the dependency wait
    pdl_wait();
    // every shared warp stages the part it reads: act = bf16(silu(gate) * up) from the shared gate_up row
    const __nv_bfloat16* grow = hs + (int64_t)m * 2 * SI;
    for (int k0 = j * 128; k0 < SI; k0 += SH_WARPS * 128)
      for (int i = lane * 8; i < 128; i += 256) {
        const uint4 gv = *reinterpret_cast<const uint4*>(grow + k0 + i);
        const uint4 uv = *reinterpret_cast<const uint4*>(grow + SI + k0 + i);
        const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w}, uw[4] = {uv.x, uv.y, uv.z, uv.w};
        uint4 av;
        uint32_t* aw = reinterpret_cast<uint32_t*>(&av);
#pragma unroll
        for (int c = 0; c < 4; ++c)
          aw[c] = pack_bf16x2(silu_mul(bf16_bits_to_float(gw[c] & 0xffffu), bf16_bits_to_float(uw[c] & 0xffffu)),
                              silu_mul(bf16_bits_to_float(gw[c] >> 16), bf16_bits_to_float(uw[c] >> 16)));
        *reinterpret_cast<uint4*>(as + xs_idx32(k0 + i)) = av;
      }
    __syncwarp();
    float acc[4][4];
    acc_zero(acc);
    auto finish = [&](int it) {
      if ((it % kpass) == kpass - 1) {
        const int tile = it / kpass;
        if (t == 0) {
          sh_part[(tile * SH_WARPS + j) * 16 + g] = acc_sum(acc, 0);
          sh_part[(tile * SH_WARPS + j) * 16 + 8 + g] = acc_sum(acc, 2);
        }
        acc_zero(acc);
      }
    };
    auto compute = [&](const BfRegs& rg, int it) {
      const int k0 = j * 128 + (it % kpass) * SH_WARPS * 128;
      if (k0 < SI) bf_compute(rg, as, k0, t, acc);
    };
    for (int it = 0; it < items; it += 2) {
      if (it + 1 < items) issue(rb, it + 1);
      compute(ra, it);
      finish(it);
      if (it + 1 < items) {
        if (it + 2 < items) issue(ra, it + 2);
        compute(rb, it + 1);
        finish(it + 1);
      }
    }
  }
  __syncthreads();
  for (int o = tid; o < 16 * TPW; o += blockDim.x) {
    const int tile = o >> 4, rr = o & 15;
    float routed = 0.f;
    for (int k = 0; k < top_k; ++k) routed += ic3[(tile * top_k + k) * 16 + rr];
    routed = bf16_round(routed);
    float y = routed;
    if (with_shared) {
      float sh = 0.f;
#pragma unroll
      for (int j = 0; j < SH_WARPS; ++j) sh += sh_part[(tile * SH_WARPS + j) * 16 + rr];
      sh = bf16_round(sh);
      const float gl = __bfloat162float(gate_logit[m]);
      const float sig = bf16_round(1.0f / (1.0f + expf(-gl)));
      const float prod = bf16_round(sh * sig);
      y = routed + prod;
    }
    out[(int64_t)m * H + n0 + o] = __float2bfloat16_rn(y);
  }
}

// ------------------------------------------------------------------------------------------------
// Dense bf16 rows x (<= 8 tokens): router logits, shared gate_up, shared gate logit in one launch.
// One CTA = one 16-row tile of one segment; 16 warps split K in slices of 128.
// ------------------------------------------------------------------------------------------------
struct DenseSeg {
  const __nv_bfloat16* w;  // [rows, H]
  __nv_bfloat16* out;      // out[m * out_stride + row]
  int rows, out_stride, tiles;
};
constexpr int DENSE_WARPS = 16;

struct DenseRegs {
  uint4 qa[4], qb[4];
};

// trigger_after_wait: raise the launch trigger once this kernel's own dependency wait has passed (everything before
// this kernel in the stream is then complete, so its successor may read such data before its own wait).
B200MOE_DEVICE void dense_rows_body(unsigned char* smem_raw, int tile, const __nv_bfloat16* __restrict__ x, int M, int H,
                                    const DenseSeg& s0, const DenseSeg& s1, const DenseSeg& s2,
                                    bool trigger_after_wait = false) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  DenseSeg seg = s0;
  if (tile >= s0.tiles) {
    tile -= s0.tiles;
    seg = s1;
    if (tile >= s1.tiles) {
      tile -= s1.tiles;
      seg = s2;
    }
  }
  const int row_stride = xs_idx32(H) + 8;  // halves; the +8 staggers token rows across banks
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);          // [8][row_stride]
  float* part = reinterpret_cast<float*>(smem_raw + (size_t)8 * row_stride * 2);  // [nwarps][16][8]

  const int ra = min(tile * 16 + g, seg.rows - 1), rb = min(tile * 16 + g + 8, seg.rows - 1);
  const __nv_bfloat16* wa = seg.w + (int64_t)ra * H;
  const __nv_bfloat16* wb = seg.w + (int64_t)rb * H;
  auto issue = [&](DenseRegs& r, int k0) {
    if (k0 < H) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        r.qa[c] = ldg_nc_keep_v4(wa + k0 + 32 * t + 8 * c);
        r.qb[c] = ldg_nc_keep_v4(wb + k0 + 32 * t + 8 * c);
      }
    }
  };
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  auto compute = [&](const DenseRegs& r, int k0) {
    if (k0 < H) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 xv = *reinterpret_cast<const uint4*>(xs + g * row_stride + xs_idx32(k0 + 32 * t + 8 * c));
        uint32_t a[4] = {r.qa[c].x, r.qb[c].x, r.qa[c].y, r.qb[c].y};
        mma_bf16_16816(acc, a, xv.x, xv.y);
        uint32_t b[4] = {r.qa[c].z, r.qb[c].z, r.qa[c].w, r.qb[c].w};
        mma_bf16_16816(acc, b, xv.z, xv.w);
      }
    }
  };
  const int kstep = nwarps * 128;
  DenseRegs r0, r1;
  issue(r0, warp * 128);          // weights depend on nothing: requested before the dependency wait
  issue(r1, warp * 128 + kstep);
  pdl_wait();
  if (trigger_after_wait) pdl_launch_dependents();
  for (int i = tid * 8; i < 8 * H; i += blockDim.x * 8) {
    const int m = i / H, k = i - m * H;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (m < M) v = *reinterpret_cast<const uint4*>(x + (int64_t)m * H + k);
    *reinterpret_cast<uint4*>(xs + m * row_stride + xs_idx32(k)) = v;
  }
  __syncthreads();
  for (int k0 = warp * 128; k0 < H; k0 += 2 * kstep) {
    compute(r0, k0);
    issue(r0, k0 + 2 * kstep);
    compute(r1, k0 + kstep);
    issue(r1, k0 + 3 * kstep);
  }
  float* mine = part + warp * 128;
  mine[g * 8 + 2 * t] = acc[0];
  mine[g * 8 + 2 * t + 1] = acc[1];
  mine[(g + 8) * 8 + 2 * t] = acc[2];
  mine[(g + 8) * 8 + 2 * t + 1] = acc[3];
  __syncthreads();
  if (tid < 128) {
    const int row = tid >> 3, m = tid & 7;
    float s = 0.f;
    for (int w = 0; w < nwarps; ++w) s += part[w * 128 + row * 8 + m];
    const int gr = tile * 16 + row;
    if (m < M && gr < seg.rows) seg.out[(int64_t)m * seg.out_stride + gr] = __float2bfloat16_rn(s);
  }
}

__global__ void __launch_bounds__(DENSE_WARPS * 32) dense_rows_kernel(const __nv_bfloat16* __restrict__ x, int M, int H,
                                                                      DenseSeg s0, DenseSeg s1, DenseSeg s2) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  dense_rows_body(smem_raw, blockIdx.x, x, M, H, s0, s1, s2, true);
}

// ------------------------------------------------------------------------------------------------
// First stage of a decode layer whose slot ids are already known (the offload path): the routed GEMM1 +
// SwiGLU and the dense rows (router logits, shared gate_up, shared gate logit) need nothing from each other,
// so they share one launch.  grid = (I / (8*NT), routes + dense_rows): CTA rows below `routes` run GEMM1 for
// one route, the rows above walk the dense 16-row tiles (tile = (y - routes) * gridDim.x + x).
// ------------------------------------------------------------------------------------------------
template <int KS>
__global__ void __launch_bounds__(G1_WARPS * 32, 2) decode_stage1_kernel(
    const __nv_bfloat16* __restrict__ x, b200moe_banks bk, const int32_t* __restrict__ ids, int routes, int top_k, int NT,
    __nv_bfloat16* __restrict__ ic2, int M, DenseSeg s0, DenseSeg s1, DenseSeg s2) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_launch_dependents();
  if ((int)blockIdx.y < routes) {
    decode_gemm1_body<KS>(smem_raw, blockIdx.x, blockIdx.y, x, bk, ids, true, nullptr, 0, nullptr, nullptr, top_k, NT, ic2);
  } else {
    const int tile = ((int)blockIdx.y - routes) * gridDim.x + blockIdx.x;
    if (tile < s0.tiles + s1.tiles + s2.tiles) dense_rows_body(smem_raw, tile, x, M, bk.hidden, s0, s1, s2);
  }
}

static int check_banks(const b200moe_banks* b) {
  if (!b || !b->gate_up || !b->gate_up_scale || !b->gate_up_global || !b->down || !b->down_scale || !b->down_global)
    return B200MOE_E_NULL;
  if (b->num_slots < 1 || b->hidden < 1 || b->intermediate < 1) return B200MOE_E_SHAPE;
  if (!aligned16(b->gate_up) || !aligned16(b->gate_up_scale) || !aligned16(b->down) || !aligned16(b->down_scale))
    return B200MOE_E_ALIGN;
  return 0;
}

struct DecodeWs {
  __nv_bfloat16 *hs, *gate_logit, *ic2, *logits;
  int64_t bytes;
};
static DecodeWs carve_decode_ws(void* ws, int M, int top_k, int I, int SI) {
  DecodeWs d;
  auto up = [](int64_t v) { return (v + 255) / 256 * 256; };
  char* p = reinterpret_cast<char*>(ws);
  int64_t off = 0;
  d.hs = reinterpret_cast<__nv_bfloat16*>(p + off); off += up((int64_t)M * 2 * SI * 2);
  d.gate_logit = reinterpret_cast<__nv_bfloat16*>(p + off); off += up((int64_t)M * 2);
  d.ic2 = reinterpret_cast<__nv_bfloat16*>(p + off); off += up((int64_t)M * top_k * I * 2);
  d.logits = reinterpret_cast<__nv_bfloat16*>(p + off); off += up((int64_t)M * 512 * 2);  // router logits scratch (E <= 512)
  d.bytes = off;
  return d;
}

static int decode_shape_ok(int M, int top_k, int H, int I, int SI) {
  if (M < 1 || M > 8 || top_k < 1 || top_k > 8) return B200MOE_E_SHAPE;
  if (H % 512 || I % 512 || H > 16384 || I > 8192) return B200MOE_E_SHAPE;
  if (SI && (SI % 128 || SI > 8192)) return B200MOE_E_SHAPE;
  return 0;
}

static int g_use_pdl = 1;

// cudaFuncSetAttribute is per device: remember (kernel, device ordinal) pairs that are done, under a lock.
static std::mutex g_attr_lock;
static std::vector<std::pair<const void*, int>> g_attr_done;
static int smem_attr_once(const void* kernel, int bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  std::lock_guard<std::mutex> guard(g_attr_lock);
  for (const auto& d : g_attr_done)
    if (d.first == kernel && d.second == dev) return 0;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return (int)e;
  g_attr_done.emplace_back(kernel, dev);
  return 0;
}

template <typename... KArgs, typename... Args>
static int launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_use_pdl ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
  return e == cudaSuccess ? 0 : (int)e;
}

static void dense_segments(const b200moe_dense* dense, __nv_bfloat16* logits, const struct DecodeWs& ws, DenseSeg (&s)[3]);

// Shape of the first-stage grid: one wave of about 256 CTAs whatever the token count, NT row tiles per CTA,
// KS = G1_WARPS / NT warps per tile along K.
struct G1Shape {
  int nt, ks, ctas_per_route;
};
static int gemm1_shape(const b200moe_banks* bk, int routes, G1Shape* g) {
  const int tiles = bk->intermediate / 8;
  const int max_ks = std::min(4, bk->hidden / FP4_SLICE);
  int cpr = 1;
  while (cpr * 2 * routes <= 256 && tiles % (cpr * 2) == 0) cpr *= 2;
  int nt = tiles / cpr;
  while (nt < G1_WARPS / max_ks && nt < tiles) nt *= 2;  // not more K shares than K slices
  if (tiles % nt) return B200MOE_E_SHAPE;
  g->nt = nt;
  g->ks = nt * 2 == G1_WARPS ? 2 : nt * 4 == G1_WARPS ? 4 : 1;
  g->ctas_per_route = tiles / nt;
  return 0;
}
static size_t gemm1_smem(int H, int nt, int ks) { return (size_t)xs_idx128(H) * 2 + (32 + 16 + (size_t)nt * ks * 16) * 4; }
static size_t dense_smem(int H, int warps) { return (size_t)8 * (xs_idx32(H) + 8) * 2 + (size_t)warps * 128 * 4; }

template <int KS>
static int launch_gemm1_ks(const __nv_bfloat16* x, const b200moe_banks* bk, const int32_t* ids, const __nv_bfloat16* logits,
                           int E, float* w_out, int32_t* ids_out, int M, int top_k, const G1Shape& g, const DecodeWs& ws,
                           cudaStream_t st) {
  if (int rc = smem_attr_once(reinterpret_cast<const void*>(&decode_gemm1_kernel<KS>), 100 * 1024)) return rc;
  return launch_k(decode_gemm1_kernel<KS>, dim3(g.ctas_per_route, M * top_k), dim3(G1_WARPS * 32),
                  gemm1_smem(bk->hidden, g.nt, KS), st, x, *bk, ids, logits, E, w_out, ids_out, top_k, g.nt, ws.ic2);
}

static int launch_gemm1(const __nv_bfloat16* x, const b200moe_banks* bk, const int32_t* ids, const __nv_bfloat16* logits,
                        int E, float* w_out, int32_t* ids_out, int M, int top_k, const DecodeWs& ws, cudaStream_t st) {
  G1Shape g;
  int rc = gemm1_shape(bk, M * top_k, &g);
  if (rc) return rc;
  if (g.ks == 2) return launch_gemm1_ks<2>(x, bk, ids, logits, E, w_out, ids_out, M, top_k, g, ws, st);
  if (g.ks == 4) return launch_gemm1_ks<4>(x, bk, ids, logits, E, w_out, ids_out, M, top_k, g, ws, st);
  return launch_gemm1_ks<1>(x, bk, ids, logits, E, w_out, ids_out, M, top_k, g, ws, st);
}

template <int KS>
static int launch_stage1_ks(const __nv_bfloat16* x, const b200moe_banks* bk, const int32_t* ids, int M, int top_k,
                            const G1Shape& g, const DecodeWs& ws, const b200moe_dense* dense, cudaStream_t st) {
  if (int rc = smem_attr_once(reinterpret_cast<const void*>(&decode_stage1_kernel<KS>), 200 * 1024)) return rc;
  DenseSeg s[3];
  dense_segments(dense, ws.logits, ws, s);
  const int routes = M * top_k, dense_tiles = s[0].tiles + s[1].tiles + s[2].tiles;
  const int dense_rows = (dense_tiles + g.ctas_per_route - 1) / g.ctas_per_route;
  const size_t smem = std::max(gemm1_smem(bk->hidden, g.nt, KS), dense_smem(bk->hidden, G1_WARPS));
  return launch_k(decode_stage1_kernel<KS>, dim3(g.ctas_per_route, routes + dense_rows), dim3(G1_WARPS * 32), smem, st, x,
                  *bk, ids, routes, top_k, g.nt, ws.ic2, M, s[0], s[1], s[2]);
}

// GEMM1 for known slot ids and the dense rows of the same layer in one launch.
static int launch_stage1(const __nv_bfloat16* x, const b200moe_banks* bk, const int32_t* ids, int M, int top_k,
                         const DecodeWs& ws, const b200moe_dense* dense, cudaStream_t st) {
  G1Shape g;
  int rc = gemm1_shape(bk, M * top_k, &g);
  if (rc) return rc;
  if (g.ks == 2) return launch_stage1_ks<2>(x, bk, ids, M, top_k, g, ws, dense, st);
  if (g.ks == 4) return launch_stage1_ks<4>(x, bk, ids, M, top_k, g, ws, dense, st);
  return launch_stage1_ks<1>(x, bk, ids, M, top_k, g, ws, dense, st);
}

static int launch_gemm2(const b200moe_banks* bk, const float* w, const int32_t* ids, int M, int top_k,
                        __nv_bfloat16* out, const DecodeWs& ws, const b200moe_dense* dense, int SI, cudaStream_t st) {
  const int H = bk->hidden, I = bk->intermediate;
  const int with_shared = dense != nullptr;
  const int si = SI > 0 ? SI : 32;
  int tpw = 1;  // row tiles per warp: about 128 CTAs whatever the token count
  while (tpw < M && (H / 16) % (tpw * 2) == 0) tpw *= 2;
  const size_t smem = (size_t)top_k * xs_idx128(I) * 2 + (size_t)xs_idx32(si) * 2 +
                      (size_t)(tpw * top_k * 16 + tpw * SH_WARPS * 16) * 4;
  if (int rc = smem_attr_once(reinterpret_cast<const void*>(&decode_gemm2_kernel), 160 * 1024)) return rc;
  const int warps = top_k + (with_shared ? SH_WARPS : 0);
  return launch_k(decode_gemm2_kernel, dim3(H / (16 * tpw), M), dim3(warps * 32), smem, st, tpw,
                  (const __nv_bfloat16*)ws.ic2, *bk, w, ids, top_k, (const __nv_bfloat16*)ws.hs,
                  with_shared ? reinterpret_cast<const __nv_bfloat16*>(dense->shared_down) : (const __nv_bfloat16*)nullptr,
                  si, (const __nv_bfloat16*)ws.gate_logit, out, with_shared);
}

// ids == nullptr: GEMM1 routes from `logits` and publishes (w_out, ids_out), which GEMM2 then reads.
static int launch_experts(const __nv_bfloat16* x, const b200moe_banks* bk, const float* w, const int32_t* ids,
                          const __nv_bfloat16* logits, int E, float* w_out, int32_t* ids_out, int M, int top_k,
                          __nv_bfloat16* out, const DecodeWs& ws, const b200moe_dense* dense, int SI, cudaStream_t st) {
  b200moe_banks nb;
  int rc = normalize_banks(bk, &nb);
  if (rc) return rc;
  bk = &nb;
  rc = launch_gemm1(x, bk, ids, logits, E, w_out, ids_out, M, top_k, ws, st);
  if (rc) return rc;
  return launch_gemm2(bk, ids != nullptr ? w : w_out, ids != nullptr ? ids : ids_out, M, top_k, out, ws, dense, SI, st);
}

static void dense_segments(const b200moe_dense* dense, __nv_bfloat16* logits, const DecodeWs& ws, DenseSeg (&s)[3]) {
  const int SI = dense->shared_intermediate, E = dense->num_experts;
  s[0] = DenseSeg{reinterpret_cast<const __nv_bfloat16*>(dense->router_w), logits, E, E, (E + 15) / 16};
  s[1] = DenseSeg{reinterpret_cast<const __nv_bfloat16*>(dense->shared_gate_up), ws.hs, 2 * SI, 2 * SI, (2 * SI + 15) / 16};
  s[2] = DenseSeg{reinterpret_cast<const __nv_bfloat16*>(dense->shared_gate), ws.gate_logit, 1, 1, 1};
}

static int launch_dense_rows(const __nv_bfloat16* x, const b200moe_dense* dense, int M, int hidden, __nv_bfloat16* logits,
                             const DecodeWs& ws, cudaStream_t st, int segment_mask = 7) {
  DenseSeg s[3];
  dense_segments(dense, logits, ws, s);
  for (int i = 0; i < 3; ++i)
    if (!(segment_mask & (1 << i))) s[i].tiles = 0;  // a segment without tiles is skipped by the tile walk
  if (s[0].tiles + s[1].tiles + s[2].tiles == 0) return 0;
  if (int rc = smem_attr_once(reinterpret_cast<const void*>(&dense_rows_kernel), 200 * 1024)) return rc;
  return launch_k(dense_rows_kernel, dim3(s[0].tiles + s[1].tiles + s[2].tiles), dim3(DENSE_WARPS * 32),
                  dense_smem(hidden, DENSE_WARPS), st, x, M, hidden, s[0], s[1], s[2]);
}

// One decode layer with known slot ids and the shared expert: two launches.
static int launch_layer_known_ids(const __nv_bfloat16* x, const b200moe_banks* bk, const float* w, const int32_t* ids, int M,
                                  int top_k, __nv_bfloat16* out, const DecodeWs& ws, const b200moe_dense* dense, int SI,
                                  cudaStream_t st) {
  b200moe_banks nb;
  int rc = normalize_banks(bk, &nb);
  if (rc) return rc;
  rc = launch_stage1(x, &nb, ids, M, top_k, ws, dense, st);
  if (rc) return rc;
  return launch_gemm2(&nb, w, ids, M, top_k, out, ws, dense, SI, st);
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int64_t b200moe_decode_workspace_bytes(int M, int top_k, int hidden, int intermediate,
                                                  int shared_intermediate, int num_experts) {
  (void)hidden;
  (void)num_experts;
  if (M < 1 || top_k < 1) return 0;
  return carve_decode_ws(nullptr, M, top_k, intermediate, shared_intermediate > 0 ? shared_intermediate : 0).bytes;
}

extern "C" int b200moe_decode_experts(const void* x, const b200moe_banks* banks, const float* topk_weights,
                                      const int32_t* topk_ids, int M, int top_k, void* out, void* workspace,
                                      int64_t workspace_bytes, void* stream) {
  int rc = check_banks(banks);
  if (rc) return rc;
  if (!x || !topk_weights || !topk_ids || !out || !workspace) return B200MOE_E_NULL;
  if ((rc = decode_shape_ok(M, top_k, banks->hidden, banks->intermediate, 0))) return rc;
  if (!aligned16(x) || !aligned16(workspace)) return B200MOE_E_ALIGN;
  DecodeWs ws = carve_decode_ws(workspace, M, top_k, banks->intermediate, 0);
  if (workspace_bytes < ws.bytes) return B200MOE_E_WORKSPACE;
  return launch_experts(reinterpret_cast<const __nv_bfloat16*>(x), banks, topk_weights, topk_ids, nullptr, 0, nullptr,
                        nullptr, M, top_k, reinterpret_cast<__nv_bfloat16*>(out), ws, nullptr, 0,
                        reinterpret_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------------------------------
// Allocation-free variant of b200moe_decode_experts.
//
// Some callers cannot hand this library a scratch buffer because they cannot allocate device memory
// where they run: a plugin slot whose host forbids cudaMalloc after start-up, code that runs while a
// caching allocator is locked (inside a stream capture or a memory-pool snapshot), or a process that
// was given its inputs and outputs by another runtime and owns no allocator at all.  For them the
// intermediate activations of the two expert GEMVs live in a fixed array inside the library image.
//
// Limits and rules:
//   * the array is B200MOE_STATIC_SCRATCH_BYTES long; every GPU that loads the library holds it until
//     the process exits.  A call whose M * top_k * intermediate needs more is refused (-6);
//   * the first call on a device looks the array's device address up (cudaGetSymbolAddress, with that
//     device current) and remembers it; make that first call outside any stream capture;
//   * every call uses the same array and it keeps the previous call's contents.  Nothing in it has to
//     start at zero: the first kernel overwrites every element the second one reads.  Two calls that
//     overlap on the GPU (different streams, no dependency) would race on it -- order them.
// Nothing here calls cudaMalloc, cudaFree or any allocating library routine.
// ------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_scratch[B200MOE_STATIC_SCRATCH_BYTES];
static void* g_static_scratch_addr[64];  // per device ordinal; written once under the lock below

static std::mutex g_static_scratch_lock;

extern "C" int b200moe_decode_experts_static(const void* x, const b200moe_banks* banks, const float* topk_weights,
                                             const int32_t* topk_ids, int M, int top_k, void* out, void* stream) {
  int rc = check_banks(banks);
  if (rc) return rc;
  if (!x || !topk_weights || !topk_ids || !out) return B200MOE_E_NULL;
  if ((rc = decode_shape_ok(M, top_k, banks->hidden, banks->intermediate, 0))) return rc;
  if (!aligned16(x)) return B200MOE_E_ALIGN;
  if (carve_decode_ws(nullptr, M, top_k, banks->intermediate, 0).bytes > (int64_t)B200MOE_STATIC_SCRATCH_BYTES)
    return B200MOE_E_STATIC_LIMIT;
  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return (int)ce;
  if (dev < 0 || dev >= 64) return B200MOE_E_DEVICE;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> guard(g_static_scratch_lock);
    if (g_static_scratch_addr[dev] == nullptr) {
      // the symbol's name is only a host-side handle; kernels need its address on THIS device
      void* p = nullptr;
      ce = cudaGetSymbolAddress(&p, g_static_scratch);
      if (ce != cudaSuccess) return (int)ce;
      if (p == nullptr) return B200MOE_E_DEVICE;
      g_static_scratch_addr[dev] = p;
    }
    scratch = g_static_scratch_addr[dev];
  }
  DecodeWs ws = carve_decode_ws(scratch, M, top_k, banks->intermediate, 0);
  return launch_experts(reinterpret_cast<const __nv_bfloat16*>(x), banks, topk_weights, topk_ids, nullptr, 0, nullptr,
                        nullptr, M, top_k, reinterpret_cast<__nv_bfloat16*>(out), ws, nullptr, 0,
                        reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_decode_block_route(const void* x, const b200moe_dense* dense, int M, int hidden, int top_k,
                                          void* logits_out, float* topk_weights, int32_t* topk_ids, void* workspace,
                                          int64_t workspace_bytes, void* stream) {
  if (!x || !dense || !dense->router_w || !dense->shared_gate_up || !dense->shared_gate || !logits_out ||
      !topk_weights || !topk_ids || !workspace)
    return B200MOE_E_NULL;
  const int SI = dense->shared_intermediate, E = dense->num_experts;
  if (M < 1 || M > 8 || hidden % 128 || hidden > 8192 || E < 1 || E > 512 || SI < 1 || top_k < 1 || top_k > E)
    return B200MOE_E_SHAPE;
  if (!aligned16(x) || !aligned16(dense->router_w) || !aligned16(dense->shared_gate_up) || !aligned16(dense->shared_gate))
    return B200MOE_E_ALIGN;
  // only hs / gate_logit are touched here; the carve is shared with stage B (I unknown here -> 0 for ic2)
  DecodeWs ws = carve_decode_ws(workspace, M, top_k, 0, SI);
  if (workspace_bytes < ws.bytes) return B200MOE_E_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int rc = launch_dense_rows(reinterpret_cast<const __nv_bfloat16*>(x), dense, M, hidden,
                             reinterpret_cast<__nv_bfloat16*>(logits_out), ws, st);
  if (rc) return rc;
  return b200moe_router_topk(logits_out, 0, E, M, E, top_k, 1, nullptr, 0, topk_weights, topk_ids, stream);
}

extern "C" int b200moe_decode_dense_rows(const void* x, const b200moe_dense* dense, int M, int hidden, int segment_mask,
                                         void* logits_out, void* workspace, int64_t workspace_bytes, void* stream) {
  if (!x || !dense || !dense->router_w || !dense->shared_gate_up || !dense->shared_gate || !workspace) return B200MOE_E_NULL;
  if ((segment_mask & 1) && !logits_out) return B200MOE_E_NULL;
  const int SI = dense->shared_intermediate, E = dense->num_experts;
  if (M < 1 || M > 8 || hidden % 128 || hidden > 8192 || E < 1 || E > 512 || SI < 1 || (segment_mask & ~7)) return B200MOE_E_SHAPE;
  if (!aligned16(x) || !aligned16(dense->router_w) || !aligned16(dense->shared_gate_up) || !aligned16(dense->shared_gate))
    return B200MOE_E_ALIGN;
  DecodeWs ws = carve_decode_ws(workspace, M, 1, 0, SI);
  if (workspace_bytes < ws.bytes) return B200MOE_E_WORKSPACE;
  return launch_dense_rows(reinterpret_cast<const __nv_bfloat16*>(x), dense, M, hidden,
                           reinterpret_cast<__nv_bfloat16*>(logits_out), ws, reinterpret_cast<cudaStream_t>(stream),
                           segment_mask);
}

extern "C" int b200moe_decode_block_experts(const void* x, const b200moe_banks* banks, const b200moe_dense* dense,
                                            const float* topk_weights, const int32_t* topk_ids, int M, int top_k,
                                            void* out, void* workspace, int64_t workspace_bytes, void* stream) {
  int rc = check_banks(banks);
  if (rc) return rc;
  if (!x || !dense || !dense->shared_down || !topk_weights || !topk_ids || !out || !workspace) return B200MOE_E_NULL;
  const int SI = dense->shared_intermediate;
  if ((rc = decode_shape_ok(M, top_k, banks->hidden, banks->intermediate, SI))) return rc;
  if (!aligned16(x) || !aligned16(workspace) || !aligned16(dense->shared_down)) return B200MOE_E_ALIGN;
  DecodeWs ws = carve_decode_ws(workspace, M, top_k, banks->intermediate, SI);
  if (workspace_bytes < ws.bytes) return B200MOE_E_WORKSPACE;
  return launch_experts(reinterpret_cast<const __nv_bfloat16*>(x), banks, topk_weights, topk_ids, nullptr, 0, nullptr,
                        nullptr, M, top_k, reinterpret_cast<__nv_bfloat16*>(out), ws, dense, SI,
                        reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_decode_block(const void* x, const b200moe_banks* banks, const b200moe_dense* dense, int M,
                                    int top_k, void* logits_out, float* topk_weights, int32_t* topk_ids, void* out,
                                    void* workspace, int64_t workspace_bytes, void* stream) {
  int rc = check_banks(banks);
  if (rc) return rc;
  if (!x || !dense || !dense->router_w || !dense->shared_gate_up || !dense->shared_down || !dense->shared_gate ||
      !logits_out || !topk_weights || !topk_ids || !out || !workspace)
    return B200MOE_E_NULL;
  const int SI = dense->shared_intermediate, E = dense->num_experts;
  if ((rc = decode_shape_ok(M, top_k, banks->hidden, banks->intermediate, SI))) return rc;
  if (E < 1 || E > 512 || top_k > E) return B200MOE_E_SHAPE;
  if (!aligned16(x) || !aligned16(workspace) || !aligned16(dense->router_w) || !aligned16(dense->shared_gate_up) ||
      !aligned16(dense->shared_down) || !aligned16(dense->shared_gate))
    return B200MOE_E_ALIGN;
  DecodeWs ws = carve_decode_ws(workspace, M, top_k, banks->intermediate, SI);
  if (workspace_bytes < ws.bytes) return B200MOE_E_WORKSPACE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  rc = launch_dense_rows(reinterpret_cast<const __nv_bfloat16*>(x), dense, M, banks->hidden,
                         reinterpret_cast<__nv_bfloat16*>(logits_out), ws, st);
  if (rc) return rc;
  return launch_experts(reinterpret_cast<const __nv_bfloat16*>(x), banks, nullptr, nullptr,
                        reinterpret_cast<const __nv_bfloat16*>(logits_out), E, topk_weights, topk_ids, M, top_k,
                        reinterpret_cast<__nv_bfloat16*>(out), ws, dense, SI, st);
}

extern "C" int b200moe_set_pdl(int enable) {
  g_use_pdl = enable ? 1 : 0;
  return 0;
}

// ------------------------------------------------------------------------------------------------
// Offload decode: one token step over a stack of MoE layers whose experts sit behind the slot cache.
// The whole per-layer sequence (host LRU, miss fills on the copy stream, event hand-over, the two decode
// launches) runs inside ONE call, so the per-layer host cost is a few microseconds of C++ instead of an
// interpreter loop.  The host never waits for the GPU here.
// ------------------------------------------------------------------------------------------------
struct b200moe_offload {
  b200moe_slot_tables tables;  // host arrays
  int num_banks, lookahead;
  std::vector<void*> dst;
  std::vector<const void*> src;  // [layer * num_banks + bank]
  std::vector<int64_t> row_bytes;
  std::vector<cudaEvent_t> filled, done;
  uint64_t calls = 0;
  // Recency list over the slots in ascending (usage, slot): the policy's victim order without a scan.  It mirrors
  // the tables as long as only this object changes them; `seen_step` detects outside changes and rebuilds it.
  std::vector<int32_t> prev, next;  // doubly linked, index S = sentinel
  int64_t seen_step = -1;
  // scratch of ensure() and of the step's plan, sized once (create) so that the launch path never allocates
  std::vector<int32_t> q, touched, miss, order, plan_src, plan_dst;
  std::vector<int> miss_n;

  void rebuild_list() {
    const int S = tables.cache_size;
    order.resize(S);
    for (int i = 0; i < S; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return tables.usage[a] < tables.usage[b]; });
    prev.assign(S + 1, S);
    next.assign(S + 1, S);
    int last = S;
    for (int i = 0; i < S; ++i) {
      next[last] = order[i];
      prev[order[i]] = last;
      last = order[i];
    }
    next[last] = S;
    prev[S] = last;
    seen_step = *tables.step;
  }
  void unlink(int s) {
    next[prev[s]] = next[s];
    prev[next[s]] = prev[s];
  }
  void push_back(int s) {
    const int S = tables.cache_size;
    prev[s] = prev[S];
    next[s] = S;
    next[prev[S]] = s;
    prev[S] = s;
  }

  // Same policy and outputs as b200moe_slot_ensure_host, O(n log n) in the number of ids instead of O(cache size).
  int ensure(int layer, const int32_t* ids, int n_ids, int32_t* ids_out, int64_t* stats) {
    b200moe_slot_tables& t = tables;
    if (seen_step != *t.step) rebuild_list();
    const int E = t.num_experts, S = t.cache_size, base = layer * E;
    const int64_t step = *t.step + 1;
    q.clear();
    for (int i = 0; i < n_ids; ++i)
      if (ids[i] >= 0 && ids[i] < E) q.push_back(ids[i]);
    std::sort(q.begin(), q.end());
    q.erase(std::unique(q.begin(), q.end()), q.end());
    touched.clear();
    miss.clear();
    for (int e : q) {
      const int slot = t.slot_for_id[base + e];
      if (slot >= 0) {
        t.usage[slot] = step;
        unlink(slot);
        touched.push_back(slot);
      } else {
        miss.push_back(e);
      }
    }
    int paired = 0;
    for (int e : miss) {
      const int v = next[S];  // least recently used untouched slot
      if (v == S) break;
      unlink(v);
      const int old = t.id_of_slot[v];
      if (old >= 0) t.slot_for_id[old] = -1;
      t.id_of_slot[v] = base + e;
      t.slot_for_id[base + e] = v;
      t.usage[v] = step;
      t.src_indices[paired] = e;
      t.evict_slots[paired] = v;
      touched.push_back(v);
      ++paired;
    }
    std::sort(touched.begin(), touched.end());  // equal usage: ascending slot
    for (int s : touched) push_back(s);
    *t.step = step;
    seen_step = step;
    *t.num_indices = paired;
    if (stats) {
      stats[0] += (int64_t)q.size();
      stats[1] += (int64_t)miss.size();
      stats[2] += 1;
    }
    for (int i = 0; i < n_ids; ++i) ids_out[i] = (ids[i] >= 0 && ids[i] < E) ? t.slot_for_id[base + ids[i]] : ids[i];
    return 0;
  }
};

extern "C" b200moe_offload* b200moe_offload_create(const b200moe_slot_tables* host_tables, int num_banks,
                                                   void* const* dst_banks, const void* const* src_banks,
                                                   const int64_t* row_bytes, int lookahead, int* err) {
  auto fail = [&](int code) -> b200moe_offload* {
    if (err) *err = code;
    return nullptr;
  };
  if (!host_tables || !dst_banks || !src_banks || !row_bytes) return fail(B200MOE_E_NULL);
  if (num_banks < 1 || lookahead < 1 || lookahead > 64 || host_tables->num_layers < 1) return fail(B200MOE_E_SHAPE);
  b200moe_offload* o = new b200moe_offload();
  o->tables = *host_tables;
  o->num_banks = num_banks;
  o->lookahead = lookahead;
  o->dst.assign(dst_banks, dst_banks + num_banks);
  o->src.assign(src_banks, src_banks + (size_t)num_banks * host_tables->num_layers);
  o->row_bytes.assign(row_bytes, row_bytes + num_banks);
  {
    const size_t cap = 64, L = (size_t)host_tables->num_layers;  // at most 8 tokens x 8 routes per layer
    o->q.reserve(cap);
    o->touched.reserve(2 * cap);
    o->miss.reserve(cap);
    o->order.reserve((size_t)host_tables->cache_size);
    o->plan_src.assign(L * cap, 0);
    o->plan_dst.assign(L * cap, 0);
    o->miss_n.assign(L, 0);
    o->prev.reserve((size_t)host_tables->cache_size + 1);
    o->next.reserve((size_t)host_tables->cache_size + 1);
  }
  o->filled.resize(lookahead + 1);
  o->done.resize(lookahead + 1);
  for (int i = 0; i <= lookahead; ++i) {
    cudaError_t e = cudaEventCreateWithFlags(&o->filled[i], cudaEventDisableTiming);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&o->done[i], cudaEventDisableTiming);
    if (e != cudaSuccess) {
      delete o;
      return fail((int)e);
    }
  }
  if (err) *err = 0;
  return o;
}

extern "C" void b200moe_offload_destroy(b200moe_offload* o) {
  if (!o) return;
  for (cudaEvent_t e : o->filled) cudaEventDestroy(e);
  for (cudaEvent_t e : o->done) cudaEventDestroy(e);
  delete o;
}

extern "C" int b200moe_offload_decode_step(b200moe_offload* o, const int32_t* routing_host, int M, int top_k,
                                           int32_t* slots_host_pinned, int32_t* slots_dev, const float* weights_dev,
                                           int64_t weights_layer_stride, const void* x, const b200moe_banks* cache,
                                           const b200moe_dense* dense, int64_t dense_layer_stride, void* out,
                                           int64_t out_layer_stride, void* workspace, int64_t workspace_bytes,
                                           int32_t* miss_src, int32_t* miss_dst, int32_t* miss_count,
                                           int64_t* h2d_bytes, void* copy_stream, void* compute_stream) {
  if (!o || !routing_host || !slots_host_pinned || !slots_dev || !weights_dev || !x || !dense || !out || !workspace)
    return B200MOE_E_NULL;
  int rc = check_banks(cache);
  if (rc) return rc;
  const int L = o->tables.num_layers, SI = dense->shared_intermediate;
  if ((rc = decode_shape_ok(M, top_k, cache->hidden, cache->intermediate, SI))) return rc;
  if (o->tables.cache_size <= M * top_k * (o->lookahead + 1)) return B200MOE_E_SHAPE;
  DecodeWs ws = carve_decode_ws(workspace, M, top_k, cache->intermediate, SI);
  if (workspace_bytes < ws.bytes) return B200MOE_E_WORKSPACE;
  cudaStream_t cs = reinterpret_cast<cudaStream_t>(copy_stream), st = reinterpret_cast<cudaStream_t>(compute_stream);
  const int n_ids = M * top_k, ring = o->lookahead + 1;
  int64_t bytes = 0;
  // plan every layer on the host first (the policy is sequential, the copies are not)
  std::vector<int>& miss_n = o->miss_n;
  std::vector<int32_t>&plan_src = o->plan_src, &plan_dst = o->plan_dst;
  for (int l = 0; l < L; ++l) {
    // stats, when given, are [L, 3]: one row per layer
    rc = o->ensure(l, routing_host + (size_t)l * n_ids, n_ids, slots_host_pinned + (size_t)l * n_ids,
                   o->tables.stats ? o->tables.stats + 3 * l : nullptr);
    if (rc) return rc;
    const int n = (int)*o->tables.num_indices;
    miss_n[l] = n;
    for (int i = 0; i < n; ++i) {
      plan_src[(size_t)l * n_ids + i] = o->tables.src_indices[i];
      plan_dst[(size_t)l * n_ids + i] = o->tables.evict_slots[i];
    }
    if (miss_count) miss_count[l] = n;
    if (miss_src) std::copy_n(&plan_src[(size_t)l * n_ids], n, miss_src + (size_t)l * n_ids);
    if (miss_dst) std::copy_n(&plan_dst[(size_t)l * n_ids], n, miss_dst + (size_t)l * n_ids);
  }
  cudaError_t ce = cudaMemcpyAsync(slots_dev, slots_host_pinned, (size_t)L * n_ids * sizeof(int32_t), cudaMemcpyHostToDevice, st);
  if (ce != cudaSuccess) return (int)ce;
  for (int l = 0; l < L; ++l, ++o->calls) {
    const int e = (int)(o->calls % ring);
    if (miss_n[l] > 0 && o->calls >= (uint64_t)o->lookahead) {
      ce = cudaStreamWaitEvent(cs, o->done[(o->calls - o->lookahead) % ring], 0);
      if (ce != cudaSuccess) return (int)ce;
    }
    if (miss_n[l] > 0) {
      rc = b200moe_slot_fill(o->num_banks, o->dst.data(), o->src.data() + (size_t)l * o->num_banks, o->row_bytes.data(),
                             &plan_dst[(size_t)l * n_ids], &plan_src[(size_t)l * n_ids], miss_n[l], cs);
      if (rc) return rc;
      for (int b = 0; b < o->num_banks; ++b) bytes += (int64_t)miss_n[l] * o->row_bytes[b];
      if ((ce = cudaEventRecord(o->filled[e], cs)) != cudaSuccess) return (int)ce;
      if ((ce = cudaStreamWaitEvent(st, o->filled[e], 0)) != cudaSuccess) return (int)ce;
    }
    // (a layer whose experts are all resident waits for nothing: its kernels follow the previous layer's under
    // programmatic dependent launch)
    const b200moe_dense* dl = reinterpret_cast<const b200moe_dense*>(reinterpret_cast<const char*>(dense) + (size_t)l * dense_layer_stride);
    rc = launch_layer_known_ids(reinterpret_cast<const __nv_bfloat16*>(x), cache, weights_dev + (size_t)l * weights_layer_stride,
                                slots_dev + (size_t)l * n_ids, M, top_k,
                                reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<char*>(out) + (size_t)l * out_layer_stride),
                                ws, dl, SI, st);
    if (rc) return rc;
    if ((ce = cudaEventRecord(o->done[e], st)) != cudaSuccess) return (int)ce;
  }
  if (h2d_bytes) *h2d_bytes += bytes;
  return 0;
}
