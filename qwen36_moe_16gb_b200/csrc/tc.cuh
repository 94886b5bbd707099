// tcgen05 / TMA / mbarrier building blocks shared by the grouped (NVFP4) and the dense (bf16) GEMM kernels (sm_100a).
#pragma once

#include <cuda.h>  // CUtensorMap (types only)

#include "common.cuh"

namespace b200moe {

B200MOE_DEVICE uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
B200MOE_DEVICE void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
B200MOE_DEVICE void mbar_arrive(uint32_t bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(bar) : "memory");
}
B200MOE_DEVICE void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
B200MOE_DEVICE uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in CTA `rank` of the cluster (shared::cluster window).
B200MOE_DEVICE uint32_t mapa_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
B200MOE_DEVICE void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
B200MOE_DEVICE void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// cta_group::2 forms: the MMA spans both CTAs of the pair, the commit arrives on the same barrier offset in every
// CTA of `mask` (an arrive, not a load), the TMA box lands in this CTA and counts its bytes on the leader's barrier.
B200MOE_DEVICE void tc_commit_pair(uint32_t bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"(mask) : "memory");
}
B200MOE_DEVICE void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, int col, int row, uint32_t leader_bar) {
  asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(col), "r"(row), "r"(leader_bar)
               : "memory");
}
// One box of a 3-D tensor -> this CTA's shared memory; completion is counted in bytes on this CTA's barrier.
B200MOE_DEVICE void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
               ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
               : "memory");
}
// One box of this CTA's shared memory -> a 2-D tensor in global memory (bulk async-group completion): commit after
// issuing, wait for the READ of shared memory before the buffer is rewritten, wait for everything before exit.
B200MOE_DEVICE void tma_store_2d(const CUtensorMap* map, uint32_t src, int col, int row) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(map), "r"(col), "r"(row), "r"(src)
               : "memory");
}
B200MOE_DEVICE void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
B200MOE_DEVICE void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
B200MOE_DEVICE void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
B200MOE_DEVICE bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}
// Bounded wait.  false = gave up (time limit, or another thread of the CTA already did).  The clock is the SM's
// cycle counter; the limit is about two seconds at 2 GHz.  mbarrier.try_wait suspends the thread until the phase
// completes or a short hardware time limit passes, so the loop itself issues few instructions.
B200MOE_DEVICE bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (int i = 0; i < 8; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > 4000000000ll) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
B200MOE_DEVICE void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
B200MOE_DEVICE void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
B200MOE_DEVICE void tc_mma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
               : "memory");
}
// (a0, a1) * (b0, b1) in one instruction (packed fp32 multiply, round to nearest: the same results as two fmul)
B200MOE_DEVICE float2 mul2(float a0, float a1, float b0, float b1) {
  unsigned long long a, b, r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
  asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "f"(b0), "f"(b1));
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  float2 o;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(o.x), "=f"(o.y) : "l"(r));
  return o;
}
// true in exactly one lane of the (converged) warp
B200MOE_DEVICE bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
B200MOE_DEVICE void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// K-major operand tile, 128-byte rows, 128B swizzle, 8-row groups 1024 B apart (tile base 1024-aligned).
B200MOE_DEVICE uint64_t umma_desc_sw128(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
B200MOE_DEVICE void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}
// 16 bytes that nobody on this SM reads again (no L1 allocation); a miss in L2 brings in the whole 128-byte line,
// because the next k-steps of the same weight row read its other sectors.
B200MOE_DEVICE uint4 ldg_nc_v4_l2line(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}
B200MOE_DEVICE uint4 lds_v4(uint32_t addr) {
  uint4 r;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "r"(addr));
  return r;
}
B200MOE_DEVICE uint32_t lds_u32(uint32_t addr) {
  uint32_t r;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(r) : "r"(addr));
  return r;
}
// Four bytes of packed E2M1 (8 codes) x one block scale (f16x2, both halves equal) -> 16 bytes of fp16, exact
B200MOE_DEVICE uint4 unpack_chunk_f16(uint32_t w, uint32_t scale2) {
  uint32_t h[4];
  e2m1x8_to_f16x2(w, h);
  return make_uint4(hmul2_u32(h[0], scale2), hmul2_u32(h[1], scale2), hmul2_u32(h[2], scale2), hmul2_u32(h[3], scale2));
}
B200MOE_DEVICE void sts_v4(uint32_t addr, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
B200MOE_DEVICE void stg_v4(void* p, const uint4& v) {
  asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// 32 contiguous bytes per lane in one instruction (address 32-byte aligned)
B200MOE_DEVICE void stg_v8(void* p, const uint32_t (&v)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]),
               "r"(v[5]), "r"(v[6]), "r"(v[7])
               : "memory");
}
// two floats -> f16x2, values beyond the fp16 range saturate to +-65504
B200MOE_DEVICE uint32_t pack_f16x2_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// 4 x 4 transpose of register blocks inside a quad of lanes (lane & 3 = j): on entry lane j holds its own blocks
// b[0..3]; on return b[k] is block j of lane k of the quad.  Two exchange rounds (lane ^ 1, lane ^ 2).
template <int NR>
B200MOE_DEVICE void quad_transpose(uint32_t (&b)[4][NR], int j) {
  const bool odd = j & 1, hi = j & 2;
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const uint32_t send = odd ? b[2 * m][r] : b[2 * m + 1][r];
      const uint32_t got = __shfl_xor_sync(0xffffffffu, send, 1);
      if (odd) b[2 * m][r] = got;
      else b[2 * m + 1][r] = got;
    }
#pragma unroll
  for (int s = 0; s < 2; ++s)
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const uint32_t send = hi ? b[s][r] : b[s + 2][r];
      const uint32_t got = __shfl_xor_sync(0xffffffffu, send, 2);
      if (hi) b[s][r] = got;
      else b[s + 2][r] = got;
    }
}

// kind::f16 instruction descriptor: D fp32, A and B fp16, both K-major, M = m (over the pair), N = n.
B200MOE_DEVICE uint32_t umma_idesc_f16(int n, int m) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// same descriptor for bf16 operands
B200MOE_DEVICE uint32_t umma_idesc_bf16(int n, int m) { return umma_idesc_f16(n, m) | (1u << 7) | (1u << 10); }
// cta_group::1 forms (one CTA owns the whole tile)
B200MOE_DEVICE void tc_mma_f16_cta(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
               : "memory");
}
B200MOE_DEVICE void tc_commit_cta(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
B200MOE_DEVICE void tma_load_2d(uint32_t dst, const CUtensorMap* map, int col, int row, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
               ::"r"(dst), "l"(map), "r"(col), "r"(row), "r"(bar)
               : "memory");
}

}  // namespace b200moe
