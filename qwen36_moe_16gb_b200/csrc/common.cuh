// Shared device helpers for the b200moe kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200moe.h"

#define B200MOE_DEVICE __device__ __forceinline__

namespace b200moe {

inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : (int)e;
}

// Dense strides filled in, every stride checked (bytes, multiples of 16, at least the dense size).
inline int normalize_banks(const b200moe_banks* in, b200moe_banks* out) {
  *out = *in;
  const int64_t h = in->hidden, i = in->intermediate;
  const int64_t dense[6] = {2 * i * (h / 2), 2 * i * (h / 16), 2 * i * 4, h * (i / 2), h * (i / 16), h * 4};
  for (int r = 0; r < 6; ++r) {
    if (out->slot_stride[r] == 0) out->slot_stride[r] = dense[r];
    if (out->slot_stride[r] < dense[r] || (out->slot_stride[r] & (r == 2 || r == 5 ? 3 : 15))) return B200MOE_E_ALIGN;
  }
  return 0;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- loads ---------------------------------------------------------------------------------------
B200MOE_DEVICE uint4 ldg_nc_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
// same sector is touched again by the next instruction of the same warp: let L1 keep it
B200MOE_DEVICE uint4 ldg_nc_keep_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}
// L2 policies for a kernel that re-reads a small array while it streams a large one through the cache: loads of the
// small array ask L2 to keep their lines, stores of the stream ask it to drop theirs first.
B200MOE_DEVICE uint64_t l2_policy_keep() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
B200MOE_DEVICE uint64_t l2_policy_stream() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
B200MOE_DEVICE uint4 ldg_nc_v4_policy(const void* p, uint64_t policy) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p), "l"(policy));
  return r;
}
B200MOE_DEVICE void stg_v4_policy(void* p, const uint4& v, uint64_t policy) {
  asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w),
               "l"(policy)
               : "memory");
}
B200MOE_DEVICE uint2 ldg_nc_v2(const void* p) {
  uint2 r;
  asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(r.x), "=r"(r.y) : "l"(p));
  return r;
}
B200MOE_DEVICE uint32_t ldg_nc_u32(const void* p) {
  uint32_t r;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(r) : "l"(p));
  return r;
}

// ---- conversions ---------------------------------------------------------------------------------
// Four bytes of packed E2M1 (8 codes, low nibble first) -> four f16x2 registers (exact).
B200MOE_DEVICE void e2m1x8_to_f16x2(uint32_t w, uint32_t (&h)[4]) {
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}
// Two e4m3 bytes (low 16 bits of s) -> f16x2 (exact).
B200MOE_DEVICE uint32_t e4m3x2_to_f16x2(uint32_t s) {
  uint32_t r;
  asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t}" : "=r"(r) : "r"(s));
  return r;
}
B200MOE_DEVICE uint32_t dup_lo16(uint32_t v) { return __byte_perm(v, v, 0x1010); }
B200MOE_DEVICE uint32_t dup_hi16(uint32_t v) { return __byte_perm(v, v, 0x3232); }
B200MOE_DEVICE uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
B200MOE_DEVICE float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
B200MOE_DEVICE float bf16_bits_to_float(uint32_t lo16) { return __uint_as_float(lo16 << 16); }
B200MOE_DEVICE uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// silu(g) * u exactly as the reference's activation kernel spells it: g / (1 + 2^(-g*log2e)) * u
B200MOE_DEVICE float silu_mul(float g, float u) {
  float e;
  asm("ex2.approx.f32 %0, %1;" : "=f"(e) : "f"(-g * 1.4426950408889634f));
  return __fdividef(g, 1.0f + e) * u;
}
// Power-of-two factor that brings a row with max |x| = amax just under the fp16 range, and its inverse.
B200MOE_DEVICE void f16_row_scale(float amax, float& scale, float& inv) {
  // amax = m * 2^e, m in [1,2): scale = 2^(14 - e)  ->  amax*scale in [2^14, 2^15)
  if (!(amax > 0.f) || !(amax < 3.0e38f)) {
    scale = 1.f;
    inv = 1.f;
    return;
  }
  int e = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
  if (e < -126) e = -126;
  int s = 14 - e;
  if (s > 126) s = 126;
  if (s < -126) s = -126;
  scale = __uint_as_float((uint32_t)(s + 127) << 23);
  inv = __uint_as_float((uint32_t)(127 - s) << 23);
}

// ---- warp MMA (register operands; used by the decode GEMVs) --------------------------------------
B200MOE_DEVICE void mma_f16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
B200MOE_DEVICE void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

B200MOE_DEVICE float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
B200MOE_DEVICE float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// b200moe_permute with one more output: inv_routes[route] = sorted position of the route (or -1); may be null.
int permute_with_inverse(const int32_t* topk_ids, int numel, int num_experts, int block, int32_t* sorted_token_ids,
                         int sorted_cap, int32_t* expert_ids, int expert_ids_cap, int32_t* num_tokens_post_pad,
                         int32_t* sorted_routes, int32_t* expert_offsets, int32_t* inv_routes, void* workspace,
                         int64_t workspace_bytes, void* stream);

}  // namespace b200moe
