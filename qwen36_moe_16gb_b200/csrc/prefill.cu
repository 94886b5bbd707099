// Prefill: grouped NVFP4 GEMMs on the 5th-generation tensor cores (tcgen05, accumulators in TMEM).
//
// One work item = (token tile of one expert, 256 weight rows), computed by a PAIR of CTAs (cluster of two,
// tcgen05 cta_group::2) as D[tokens x 256 weight rows] += A[tokens x 64] * B[256 x 64]^T per k-step, kind::f16
// with fp16 operands, fp32 accumulation.
//   A = token rows, fp16.  They are contiguous: a pre-pass copies x into expert order (one warp per token writes the
//       row to the sorted position of each of its routes), scaled per row by a power of two into fp16 range (exact;
//       the epilogue multiplies the inverse back); the
//       down GEMM reads the ic2 rows the gate_up GEMM wrote, already in expert order.  One thread per CTA asks the
//       TMA unit for boxes of 64 rows x 64 k (128-byte swizzle).  Each CTA of the pair holds its own token rows:
//       128 of a 256-token tile, or 64 of a tile with at most 128 tokens (M = 128 over the pair costs half the
//       tensor time of M = 256).
//   B = weight rows.  Each CTA unpacks 128 of the item's 256 rows: E2M1 codes -> f16x2 (cvt), times the E4M3 block
//       scale converted to f16x2 (one multiply, exact: at most 6 significant bits, range 2^-10 .. 2688), stored
//       into the 128-byte-swizzled K-major layout the MMA descriptor describes.  The packed bytes and scales
//       come through a staging ring in shared memory that a second TMA thread fills four k-steps at a time
//       (128 contiguous bytes of every row), so the unpack warps never have a global load in flight: a warp
//       whose threads each read their own row from global memory touches 32 cache lines per instruction, and
//       the SM's load/store pipe (one line per cycle, shared with every shared-memory store) was the bottleneck
//       of that form; a proxy fence or barrier arrive also waits for the thread's loads.
//   D   TMEM lane = token, column = weight row: an epilogue thread owns ONE token and reads consecutive output
//       columns, so SwiGLU pairs sit in one thread (gate and up rows interleave inside an item).  gate_up: four
//       lanes exchange their pieces before they store, so that one store instruction writes whole sectors.  down:
//       the per-route rows stay in (padded) expert order, a warp's 32 rows are consecutive, and they leave by TMA
//       store from a swizzled staging tile; rows bound for another GPU or wanted in route order take the exchange
//       + store path.  The fp32 per-row global, the SwiGLU and the router weight are applied here with the
//       reference's bf16 rounding points.
// The MMA time of an instruction is proportional to N and independent of M (measured: 128 cycles for N = 256,
// 64 for N = 128, for M = 128 as for M = 64 rows per CTA), so weights fill N and the tokens stream through M.
//
// Warp roles (one persistent CTA pair per two SMs, static round-robin over the item list):
//   epilogue warps   (4 gate_up, 16 down) TMEM -> registers -> global; warp w may touch TMEM lanes 32 (w % 4) .. +31
//   unpack warps     groups of four (4 groups gate_up, 2 down); group g fills the B slot of the k-steps with index
//                    = g mod groups, one thread per weight row (64 k = 32 packed bytes + 4 scales); every warp
//                    tells the pair leader's barrier itself that its rows of the k-step are stored
//   token TMA warp   lane 0 posts the byte count (leader) and issues this CTA's token boxes
//   weight TMA warp  lane 0 fills the packed-weight staging ring of this CTA
//   table warp       fetches an item's 256 per-column globals into a shared-memory table, up to two items ahead
//   MMA warp         one elected lane of the pair's leader issues tcgen05.mma / tcgen05.commit; the warp owns the TMEM
// Every mbarrier wait is bounded: on time-out the CTA records a status word, stops, frees its TMEM.
#include <algorithm>
#include <cstdlib>
#include <mutex>

#include <cuda.h>  // CUtensorMap (types only; the encoder is looked up at run time)

#include "common.cuh"
#include "tc.cuh"

namespace b200moe {

constexpr int BK = 64;
constexpr int TOK_ROWS = 128;                        // token rows a CTA holds per k-step (64 used in the half form)
constexpr int WROWS = 128;                           // weight rows a CTA unpacks per k-step
constexpr int ITEM_N = 2 * WROWS;                    // weight rows per item (the MMA's N)
constexpr int TN = 2 * TOK_ROWS;                     // tokens per full tile
constexpr int A_BYTES = TOK_ROWS * BK * 2, B_BYTES = WROWS * BK * 2;
#ifndef B200MOE_ST1
#define B200MOE_ST1 4
#endif
constexpr int GROUP_WARPS = 4;                       // an unpack group: one thread per weight row of a k-step
constexpr int SUPER = 4;                             // k-steps per staged weight block: 128 packed bytes of every row
constexpr int W_PACKED_BYTES = WROWS * (SUPER * BK / 2), W_SCALE_BYTES = WROWS * (SUPER * BK / 16);
constexpr int W_BYTES = W_PACKED_BYTES + W_SCALE_BYTES;
// Ring depths.  One slot per k-step holds the token rows and the unpacked weight rows (one tcgen05.commit frees
// both): five k-steps; staged packed weights: three blocks of four k-steps.
constexpr int ST_MAX = 5, SW = 3;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;
static_assert(GROUP_WARPS * 32 == WROWS, "one unpack thread per weight row of a k-step");
static_assert(W_PACKED_BYTES % 1024 == 0 && W_BYTES % 1024 == 0, "swizzled tiles start on 1024-byte boundaries");

// Warp roles by mode (0 = gate_up + SwiGLU, 1 = down x router weight).  gate_up has 32 k-steps per item and half an
// output per weight row: four unpack groups (group g owns the k-steps with index = g mod 4) keep the MMA fed and
// four epilogue warps drain it.  The down GEMM has eight k-steps per item and 128 KB of output per item: what the
// MMA waits for is the epilogue, a latency chain per warp (TMEM load, convert, quad exchange, store), so it gets
// sixteen epilogue warps (four per TMEM lane quarter, 64 columns each) and two unpack groups.
template <int MODE>
struct Roles {
  static constexpr int EPI = MODE == 0 ? 4 : 16;
  static constexpr int GROUPS = MODE == 0 ? 4 : 2;
  static constexpr int ST = MODE == 0 ? 5 : B200MOE_ST1;   // operand ring slots (one k-step each)
  static constexpr int UNPACK_WARPS = GROUPS * GROUP_WARPS;
  static constexpr int UNPACK0 = EPI, TMA_A = EPI + UNPACK_WARPS, TMA_W = TMA_A + 1, TABLE = TMA_W + 1, MMA = TABLE + 1;
  static constexpr int THREADS = (MMA + 1) * 32;
  static_assert(SUPER % GROUPS == 0, "a group visits every staged block the same number of times");
};

struct GgParams {
  CUtensorMap a_map;             // token rows [positions, K] fp16 as 64-column x 64-row boxes, 128B swizzle
  CUtensorMap w_map;             // packed weights [slots, N, K/2] bytes as 128-byte x 64-row boxes, 128B swizzle
  CUtensorMap s_map;             // block scales [slots, N, K/16] bytes as 16-byte x 64-row boxes
  const uint8_t* packed;         // [slots, N, K/2]
  const uint8_t* scales;         // [slots, N, K/16]
  const float* globals;          // [slots, N]
  int64_t packed_stride, scale_stride, global_stride;  // bytes from one slot to the next
  int N, K, NT;                  // weight rows, reduction length, items per token tile
  int half_n;                    // mode 0: intermediate size (gate rows [0, half_n), up rows [half_n, N))
  int w_staged;                  // 1: packed weights come through the staging ring (K a multiple of 256)
  const int4* mtiles;            // {slot, first sorted position, rows, 1 if the tile runs in the half form}
  const int32_t* num_mtiles;
  const int32_t* sorted_routes;  // sorted position -> flat route id
  const float* topk_w;           // [routes]
  const float* w_sorted;         // mode 1: router weight by sorted position
  const float* a_inv;            // mode 0: inverse of the power-of-two scale of every token row
  void* out;                     // mode 0: ic2 [pos, half_n] fp16; mode 1: ic3 bf16, [route, N] or [pos, N] (out_sorted)
  CUtensorMap o_map;             // mode 1, out_sorted: ic3 [pos, N] as 32-column x 32-row boxes, 64B swizzle
  int out_sorted;                // mode 1: rows go to their sorted position + pad_off[slot], 32-row groups by TMA store
  const int32_t* pad_off;        // [slots]: shift of a slot's rows in the padded expert order
  __nv_bfloat16* const* out_peers;  // mode 1, expert parallel: ic3 of every rank (peer-mapped), or null
  int routes_per_rank;           // global route g belongs to rank g / routes_per_rank
  int64_t route_offset;          // global route = (local route + route_offset) mod total_routes: a call covers a slice of
  int64_t total_routes;          // the box's tokens, which may wrap from the last rank's tokens to the first's
  int32_t* status;
};

struct alignas(16) GgShared {
  unsigned long long full[ST_MAX], empty[ST_MAX], full_w[SW], empty_w[SW];
  unsigned long long tmem_full[2], tmem_empty[2], table[2], table_empty[2];
  uint32_t tmem_base;
  int abort_flag;
  alignas(16) float gl[2][ITEM_N];  // per accumulator buffer: the fp32 global of every column of the item
};
constexpr size_t GG_SMEM = 1024 + (size_t)ST_MAX * STAGE_BYTES + (size_t)SW * W_BYTES + sizeof(GgShared);

// Cycle accounting of the roles of CTA 0 (diagnostic build, -DB200MOE_GG_PROFILE): every role adds up the cycles
// it spends in its waits and in its work; read back with b200moe_debug_gg_profile.
#ifdef B200MOE_GG_PROFILE
__device__ long long g_gg_prof[2][32];
__device__ unsigned long long g_gg_pairs[2][2][160];   // [mode][start | end][CTA]: globaltimer, ns
B200MOE_DEVICE unsigned long long gtimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define PROF_DECL(n) long long prof[n] = {};
#define PROF_T(var) const long long var = clock64();
#define PROF_ADD(slot, a, b) prof[slot] += (b) - (a);
#define PROF_OUT(base, n) if (blockIdx.x == 0) for (int i_ = 0; i_ < (n); ++i_) g_gg_prof[MODE][(base) + i_] = prof[i_];
#else
#define PROF_DECL(n)
#define PROF_T(var)
#define PROF_ADD(slot, a, b)
#define PROF_OUT(base, n)
#endif

template <int MODE>
__global__ void __launch_bounds__(Roles<MODE>::THREADS, 1) grouped_gemm_kernel(const __grid_constant__ GgParams p) {
  using R = Roles<MODE>;
  constexpr int EPI_WARPS = R::EPI;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  constexpr int ST = R::ST;
  GgShared* sh = reinterpret_cast<GgShared*>(ring + (size_t)ST_MAX * STAGE_BYTES + (size_t)SW * W_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ring_u32 = smem_u32(ring), ring_w = ring_u32 + ST * STAGE_BYTES;
  volatile int* abort_flag = &sh->abort_flag;
  const int rank = (int)cluster_ctarank();
  const int unit = (int)(blockIdx.x >> 1), units = (int)(gridDim.x >> 1);

#ifdef B200MOE_GG_PROFILE
  if (tid == 0 && blockIdx.x < 160) g_gg_pairs[MODE][0][blockIdx.x] = gtimer();
  const long long clk_start = clock64();
#endif
  if (tid == 0) {
    for (int s = 0; s < ST; ++s) {
      // the leader's byte-count arrive (+ the bytes of both CTAs) and every unpack warp of the k-step's group in both CTAs
      mbar_init(smem_u32(&sh->full[s]), 1 + 2 * GROUP_WARPS);
      mbar_init(smem_u32(&sh->empty[s]), 1);             // the MMA thread's commit
    }
    for (int s = 0; s < SW; ++s) {
      mbar_init(smem_u32(&sh->full_w[s]), 1);            // the weight TMA thread's byte-count arrive (+ bytes)
      mbar_init(smem_u32(&sh->empty_w[s]), R::UNPACK_WARPS * (SUPER / R::GROUPS));  // one arrival per unpack warp and visit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->table[b]), 1);                 // the table warp has filled gl[b]
      mbar_init(smem_u32(&sh->table_empty[b]), EPI_WARPS);   // every epilogue warp has read gl[b] for the last time
      mbar_init(smem_u32(&sh->tmem_full[b]), 1);
      mbar_init(smem_u32(&sh->tmem_empty[b]), 2 * EPI_WARPS);
    }
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == R::MMA) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)),
                 "r"((uint32_t)TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the other CTA's barriers exist before anyone arrives on them
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const int NT = p.NT;
  const int total_items = (*p.num_mtiles) * NT;
  const int KB = p.K / BK;
  const int my_items = total_items > unit ? (total_items - unit + units - 1) / units : 0;
  const uint32_t total_steps = (uint32_t)my_items * (uint32_t)KB;  // k-steps of this pair over all its items
  auto leader = [&](const unsigned long long* bar) { return mapa_rank(smem_u32(bar), 0); };
  // weight row (of the slot's matrix) behind row j of item column order: gate_up items interleave gate and up
  auto weight_row = [&](int wt, int j) {
    if (MODE == 0) return (j & 1) ? p.half_n + wt * (ITEM_N / 2) + (j >> 1) : wt * (ITEM_N / 2) + (j >> 1);
    return wt * ITEM_N + j;
  };

  if (warp < EPI_WARPS) {
    // ------------------------------------------------------------------ epilogue
    // warp w: TMEM lanes 32 (w % 4) .. +31 (the lanes a warp may touch); with eight warps, w / 4 picks the column half
    const int q = warp & 3, hsel = warp >> 2, jq = lane & 3;
    constexpr int CH = EPI_WARPS / 4;
    constexpr int NR = MODE == 0 ? 4 : 8;   // registers of one 16-column chunk after conversion (8 fp16 / 16 bf16)
    int tl = 0;
    PROF_DECL(6)
    for (int item = unit; item < total_items; item += units, ++tl) {
      PROF_T(p0)
      const int tt = item / NT, wt = item - tt * NT;
      const int4 info = p.mtiles[tt];
      const int buf = tl & 1, rows = info.z, half = info.w;
      // full form: lane = token rank*128 + lane, columns = weight rows; half form: lanes 0..63 hold tokens
      // rank*64 + lane with weight rows 0..127, lanes 64..127 the same tokens with weight rows 128..255
      const int tok = half ? rank * 64 + (q & 1) * 32 + lane : rank * TOK_ROWS + q * 32 + lane;
      // the warps of a lane quarter split the columns in pieces of at least 64 (the unit of the quad exchange below):
      // a half-form tile has 128 columns per lane, which keeps two of them busy
      const int ch = (half && CH > 2) ? 2 : CH;
      const int ncols = hsel < ch ? (half ? ITEM_N / 2 : ITEM_N) / ch : 0;   // TMEM columns of this warp
      const int col0 = hsel * ncols;
      const int n_base = col0 + (half ? (q >> 1) * (ITEM_N / 2) : 0);  // item column behind TMEM column col0
      const bool valid = tok < rows && ncols > 0;
      const int pos = info.y + (valid ? tok : 0);
      // mode 0: inverse token scale; mode 1: router weight -- both by sorted position
      const float mul = (MODE == 0 ? p.a_inv : p.w_sorted)[pos];
      // the item's per-column globals are in gl[buf] once the table warp says so (bounded wait)
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->table[buf]), (tl >> 1) & 1, abort_flag))) break;
      char* dst = nullptr;      // first byte of this thread's outputs for item column n_base; null = no token here
      if (MODE == 0) {
        dst = reinterpret_cast<char*>(p.out) + ((int64_t)pos * p.half_n + wt * (ITEM_N / 2) + (n_base >> 1)) * 2;
      } else if (!p.out_sorted) {
        const int route = p.sorted_routes[pos];
        __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(p.out) + (int64_t)route * p.N;
        if (p.out_peers != nullptr) {  // the row goes straight to the token's home GPU over NVLink
          int64_t groute = route + p.route_offset;
          if (groute >= p.total_routes) groute -= p.total_routes;
          const int home = (int)(groute / p.routes_per_rank);
          base = p.out_peers[home] + (groute - (int64_t)home * p.routes_per_rank) * p.N;
        }
        dst = reinterpret_cast<char*>(base + wt * ITEM_N + n_base);
      }
      if (!valid) dst = nullptr;
      PROF_T(e0)
      PROF_ADD(3, p0, e0)
      const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->tmem_full[buf]), (tl >> 1) & 1, abort_flag));
      if (!ok) break;
      PROF_T(e1)
      tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * ITEM_N + col0);
      const float* glt = &sh->gl[buf][n_base];
      // one chunk = 16 TMEM columns of this thread's token -> NR registers of output
      auto convert = [&](const uint32_t (&v)[16], int c, uint32_t (&o)[NR]) {
        const float4* g4 = reinterpret_cast<const float4*>(glt + c);
        if (MODE == 0) {
          // columns 2i / 2i+1 = gate / up of output c/2 + i
          float y[8];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 g = g4[i];  // gate, up, gate, up
            float2 a = mul2(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), mul, mul);
            float2 b = mul2(__uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]), mul, mul);
            a = mul2(a.x, a.y, g.x, g.y);
            b = mul2(b.x, b.y, g.z, g.w);
            y[2 * i] = bf16_round(silu_mul(bf16_round(a.x), bf16_round(a.y)));
            y[2 * i + 1] = bf16_round(silu_mul(bf16_round(b.x), bf16_round(b.y)));
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) o[i] = pack_f16x2_sat(y[2 * i], y[2 * i + 1]);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 g = g4[i];
            float2 a = mul2(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]), g.x, g.y);
            float2 b = mul2(__uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]), g.z, g.w);
            a = mul2(a.x, a.y, mul, mul);
            b = mul2(b.x, b.y, mul, mul);
            o[2 * i] = pack_bf16x2(a.x, a.y);
            o[2 * i + 1] = pack_bf16x2(b.x, b.y);
          }
        }
      };
      // Down GEMM with rows in (padded) expert order: a warp with at least one real route among its 32 tile rows owns
      // a 32 x 64 box of consecutive rows of ic3 (an expert's segment is padded to a multiple of 32 rows).  It converts chunk by chunk into its staging tile (row = lane, 16-byte chunks
      // swizzled by the row like a TMA tile, so the stores hit every bank once) and one lane hands the tile to a TMA
      // store: no exchange between lanes and no store instructions in the chain.  The staging tile is rewritten only
      // after the previous store has read it.  (The 32 KB of staging tiles cost this GEMM one of its ring slots.)
      bool by_tma = false;
      if constexpr (MODE == 1) by_tma = p.out_sorted && ncols > 0 && tok - lane < rows;
      if (by_tma) {
        // two halves of 32 columns through one 2 KB staging tile (64-byte rows, 64B swizzle): the first half's store
        // has long read the tile when the second half is converted
        const uint32_t stage = ring_u32 + ST * STAGE_BYTES + SW * W_BYTES + warp * 2048;
        const uint32_t srow = stage + lane * 64, sx = (lane >> 1) & 3;
        const int out_row0 = info.y + p.pad_off[info.x] + tok - lane;   // rows past the tile's end land in the padding
        uint32_t v[16];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
          for (int ii = 0; ii < 2; ++ii) {
            tc_ld16(tbase + 32 * hh + 16 * ii, v);
            tc_wait_ld();
            uint32_t o[NR];
            convert(v, 32 * hh + 16 * ii, o);
            if (ii == 0) {
              if (lane == 0) bulk_wait_read_all();
              __syncwarp();
            }
            sts_v4(srow + (((2 * ii) ^ sx) << 4), make_uint4(o[0], o[1], o[2], o[3]));
            sts_v4(srow + (((2 * ii + 1) ^ sx) << 4), make_uint4(o[NR - 4], o[NR - 3], o[NR - 2], o[NR - 1]));
          }
          if (hh == 1) tc_fence_before();
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (hh == 1) {
              mbar_arrive_cluster(leader(&sh->tmem_empty[buf]));
              mbar_arrive(smem_u32(&sh->table_empty[buf]));
            }
            tma_store_2d(&p.o_map, stage, wt * ITEM_N + n_base + 32 * hh, out_row0);
            bulk_commit();
          }
        }
        PROF_T(e2)
        PROF_ADD(0, e0, e1) PROF_ADD(1, e1, e2) PROF_ADD(2, 0, 1)
        continue;
      }
      // 64 columns at a time: four chunks, exchanged inside the quad so that lane j holds piece j of the outputs
      // of each of the quad's four tokens; a store instruction then covers contiguous pieces of eight tokens
#pragma unroll 1
      for (int c = 0; c < ncols; c += 64) {
        uint32_t blk[4][NR];
        uint32_t v[16];
        PROF_T(g0)
        if constexpr (MODE == 0) {
          // two TMEM loads per wait; the second pair is in flight while the first is converted (the down GEMM's
          // epilogue has no registers to spare for the second buffer)
          uint32_t v2[16];
          tc_ld16(tbase + c, v);
          tc_ld16(tbase + c + 16, v2);
          tc_wait_ld();
          convert(v, c, blk[0]);
          tc_ld16(tbase + c + 32, v);
          convert(v2, c + 16, blk[1]);
          tc_ld16(tbase + c + 48, v2);
          tc_wait_ld();
          convert(v, c + 32, blk[2]);
          convert(v2, c + 48, blk[3]);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            tc_ld16(tbase + c + 16 * i, v);
            tc_wait_ld();
            convert(v, c + 16 * i, blk[i]);
          }
        }
        PROF_T(g1)
        quad_transpose<NR>(blk, jq);
        PROF_T(g2)
        PROF_ADD(3, g0, g1) PROF_ADD(4, g1, g2)
        // bytes of 64 columns per token: 64 (mode 0, fp16 outputs of 32 pairs) or 128 (mode 1)
        const int gbyte = MODE == 0 ? c : 2 * c;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // destination of token k of this lane's quad
          char* dk = reinterpret_cast<char*>(__shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)dst, (lane & ~3) + k));
          if (dk == nullptr) continue;
          // lane j of the quad writes piece j of token k: 16 (mode 0) or 32 (mode 1) contiguous bytes, whole sectors
          char* d = dk + gbyte + jq * (NR * 4);
          if constexpr (NR == 8) stg_v8(d, blk[k]);
          else stg_v4(d, make_uint4(blk[k][0], blk[k][1], blk[k][2], blk[k][3]));
        }
      }
      PROF_T(e15)
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive_cluster(leader(&sh->tmem_empty[buf]));
        mbar_arrive(smem_u32(&sh->table_empty[buf]));
      }
      PROF_T(e2)
      PROF_ADD(0, e0, e1) PROF_ADD(1, e1, e2) PROF_ADD(2, 0, 1) PROF_ADD(5, e15, e2)
    }
    if (MODE == 1 && lane == 0) bulk_wait_all();   // this warp's TMA stores have left shared memory and landed
    if (tid == 0) { PROF_OUT(0, 3) }
#ifdef B200MOE_GG_PROFILE
    if (tid == 0 && blockIdx.x == 0) for (int i_ = 3; i_ < 6; ++i_) g_gg_prof[MODE][13 + i_] = prof[i_];
#endif
  } else if (warp < R::TMA_A) {
    // ------------------------------------------------------------------ weight unpackers
    constexpr int GROUPS = R::GROUPS;
    // thread -> weight row `l` of this CTA's half of the item, all 64 k of a k-step: 32 packed bytes, four block scales
    const int u = warp - R::UNPACK0, grp = u / GROUP_WARPS, l = (u % GROUP_WARPS) * 32 + lane;
    const int j = rank * WROWS + l;  // row inside the item
    const uint32_t b_row = l * 128, b_x = l & 7;
    PROF_DECL(4)
    // One row of a k-step: unpack, wait for the slot, store, fence, tell the leader.  gate_up unpacks into registers
    // BEFORE it waits (the wait -> store -> fence -> arrive chain is what the MMA thread waits for); down, with 28
    // warps and 72 registers per thread, unpacks chunk by chunk after the wait.  `release` runs once the packed
    // registers have been consumed (the staged path frees its block there).
    constexpr bool PRE_UNPACK = MODE == 0;   // the down GEMM's 72 registers per thread do not hold the unpacked row
    auto produce_row = [&](uint32_t it, const uint4& q0, const uint4& q1, uint32_t sc, auto release) -> bool {
      const int s = it % ST;
      const uint32_t s01 = e4m3x2_to_f16x2(sc & 0xffffu), s23 = e4m3x2_to_f16x2(sc >> 16);
      const uint32_t sc0 = dup_lo16(s01), sc1 = dup_hi16(s01), sc2 = dup_lo16(s23), sc3 = dup_hi16(s23);
      const uint32_t w[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
      const uint32_t sw[4] = {sc0, sc1, sc2, sc3};
      uint4 c[8];
      if (PRE_UNPACK) {
#pragma unroll
        for (int i = 0; i < 8; ++i) c[i] = unpack_chunk_f16(w[i], sw[i >> 1]);
        release();
      }
      PROF_T(u0)
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->empty[s]), ((it / ST) & 1) ^ 1, abort_flag))) return false;
      PROF_T(u1)
      PROF_ADD(1, u0, u1)
      const uint32_t sb = ring_u32 + s * STAGE_BYTES + A_BYTES + b_row;
#pragma unroll
      for (int i = 0; i < 8; ++i) sts_v4(sb + ((i ^ b_x) << 4), PRE_UNPACK ? c[i] : unpack_chunk_f16(w[i], sw[i >> 1]));
      if (!PRE_UNPACK) release();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(leader(&sh->full[s]));
      return true;
    };
    if (p.w_staged) {
      // The packed bytes of four k-steps of every row sit in a staged block: rows in box order (gate_up: 64 gate
      // rows, then 64 up rows), 128 bytes each, 16-byte chunks swizzled by the row; k-step kk of the block is chunk
      // pair (2 kk, 2 kk + 1).  Scales: 16 bytes per row after the packed part, four per k-step.
      const int tr = MODE == 0 ? ((l & 1) ? 64 + (l >> 1) : (l >> 1)) : l;
      for (uint32_t it = grp; it < total_steps; it += GROUPS) {
        const uint32_t blk = it / SUPER, kk = it % SUPER;   // k-step kk of the block: chunk pair (2 kk, 2 kk + 1)
        const uint32_t w_off0 = tr * 128 + (((2 * kk) ^ (tr & 7)) << 4), w_off1 = tr * 128 + (((2 * kk + 1) ^ (tr & 7)) << 4);
        const uint32_t s_off = W_PACKED_BYTES + tr * 16 + kk * 4;
        const int ws = blk % SW;
        PROF_T(w0)
        if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->full_w[ws]), (blk / SW) & 1, abort_flag))) break;
        PROF_T(w1)
        PROF_ADD(0, w0, w1) PROF_ADD(3, 0, 1)
        const uint32_t wb = ring_w + ws * W_BYTES;
        const uint4 q0 = lds_v4(wb + w_off0), q1 = lds_v4(wb + w_off1);
        const uint32_t sc = lds_u32(wb + s_off);
        const bool stored = produce_row(it, q0, q1, sc, [&]() {
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sh->empty_w[ws]));  // every lane has consumed its part of the block
        });
        if (!stored) break;
        PROF_T(w2)
        PROF_ADD(2, w1, w2)
      }
      if (tid == R::UNPACK0 * 32) { PROF_OUT(4, 4) }
    } else {
      // Reductions that are not a multiple of 256 (small test shapes): every thread reads its row from global memory,
      // three of its steps ahead.  The loop is unrolled over the three register sets, so a set is only read again
      // three steps after its loads were issued.
      int l_item = unit, l_kb = grp;  // (item, k-step) of the next request
      const uint8_t *lprow = nullptr, *lsrow = nullptr;
      auto place = [&]() {
        while (l_kb >= KB) {
          l_kb -= KB;
          l_item += units;
        }
        if (l_item >= total_items) return;
        const int tt = l_item / NT, wt = l_item - tt * NT;
        const int slot = p.mtiles[tt].x;
        const int wrow = weight_row(wt, j);
        lprow = p.packed + (int64_t)slot * p.packed_stride + (int64_t)wrow * (p.K >> 1);
        lsrow = p.scales + (int64_t)slot * p.scale_stride + (int64_t)wrow * (p.K >> 4);
      };
      place();
      struct WRegs {
        uint4 q0, q1;
        uint32_t sc;
      };
      auto fetch = [&](WRegs& r) {
        if (l_item < total_items) {
          r.q0 = ldg_nc_v4_l2line(lprow + l_kb * 32);
          r.q1 = ldg_nc_v4_l2line(lprow + l_kb * 32 + 16);
          r.sc = ldg_nc_u32(lsrow + l_kb * 4);
          l_kb += GROUPS;
          if (l_kb >= KB) place();
        }
      };
      auto step = [&](WRegs& r, uint32_t it) -> bool {
        if (!produce_row(it, r.q0, r.q1, r.sc, []() {})) return false;
        fetch(r);
        return true;
      };
      WRegs r0{}, r1{}, r2{};
      fetch(r0);
      fetch(r1);
      fetch(r2);
      for (uint32_t it = grp; it < total_steps; it += 3 * GROUPS) {
        if (!step(r0, it)) break;
        if (it + GROUPS < total_steps && !step(r1, it + GROUPS)) break;
        if (it + 2 * GROUPS < total_steps && !step(r2, it + 2 * GROUPS)) break;
      }
    }
  } else {
   if (warp == R::TMA_A) {
    // ------------------------------------------------------------------ token rows (A operand)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      int4 info_next = unit < total_items ? p.mtiles[unit / NT] : make_int4(0, 0, 0, 0);
      for (int item = unit; item < total_items && ok; item += units) {
        const int4 info = info_next;
        if (item + units < total_items) info_next = p.mtiles[(item + units) / NT];  // needed one item from now
        const int half = info.w;
        const int row0 = info.y + rank * (half ? 64 : TOK_ROWS);
        const int boxes = half ? 1 : 2;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % ST;
          ok = mbar_wait(smem_u32(&sh->empty[s]), ((it / ST) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t sa = ring_u32 + s * STAGE_BYTES;
          const uint32_t bar = leader(&sh->full[s]);
          if (rank == 0) mbar_arrive_expect_tx(smem_u32(&sh->full[s]), 2u * (uint32_t)boxes * (64u * 128u));
          for (int b = 0; b < boxes; ++b) tma_load_2d_pair(sa + b * (64 * 128), &p.a_map, kb * BK, row0 + b * 64, bar);
        }
      }
    }
  } else if (warp == R::TMA_W) {
    // ------------------------------------------------------------------ packed weights -> staging ring
    if (lane == 0 && p.w_staged) {
      uint32_t blk = 0;
      bool ok = true;
      int slot_next = unit < total_items ? p.mtiles[unit / NT].x : 0;
      const int blocks = KB / SUPER;
      for (int item = unit; item < total_items && ok; item += units) {
        const int slot = slot_next, wt = item % NT;
        if (item + units < total_items) slot_next = p.mtiles[(item + units) / NT].x;  // needed one item from now
        // first row of the two 64-row boxes of this CTA's half of the item
        int row_a, row_b;
        if (MODE == 0) {
          row_a = wt * (ITEM_N / 2) + 64 * rank;
          row_b = p.half_n + row_a;
        } else {
          row_a = wt * ITEM_N + WROWS * rank;
          row_b = row_a + 64;
        }
        for (int ss = 0; ss < blocks; ++ss, ++blk) {
          const int ws = blk % SW;
          ok = mbar_wait(smem_u32(&sh->empty_w[ws]), ((blk / SW) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t wb = ring_w + ws * W_BYTES, bar = smem_u32(&sh->full_w[ws]);
          mbar_arrive_expect_tx(bar, (uint32_t)W_BYTES);
          tma_load_3d(wb, &p.w_map, ss * (SUPER * BK / 2), row_a, slot, bar);
          tma_load_3d(wb + W_PACKED_BYTES / 2, &p.w_map, ss * (SUPER * BK / 2), row_b, slot, bar);
          tma_load_3d(wb + W_PACKED_BYTES, &p.s_map, ss * (SUPER * BK / 16), row_a, slot, bar);
          tma_load_3d(wb + W_PACKED_BYTES + W_SCALE_BYTES / 2, &p.s_map, ss * (SUPER * BK / 16), row_b, slot, bar);
        }
      }
    }
  } else if (warp == R::TABLE) {
    // ------------------------------------------------------------------ table warp: per-column globals of an item -> gl[buf]
    // (two items ahead of the epilogue at most; the epilogue warps only wait for it, not for one another)
    int tlr = 0;
    for (int item = unit; item < total_items; item += units, ++tlr) {
      const int buf = tlr & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->table_empty[buf]), ((tlr >> 1) & 1) ^ 1, abort_flag))) break;
      const int tt = item / NT, wt = item - tt * NT;
      const float* gsrc = p.globals + (int64_t)p.mtiles[tt].x * (p.global_stride >> 2);
      float g[ITEM_N / 32];
#pragma unroll
      for (int i = 0; i < ITEM_N / 32; ++i) g[i] = gsrc[weight_row(wt, lane + 32 * i)];
#pragma unroll
      for (int i = 0; i < ITEM_N / 32; ++i) sh->gl[buf][lane + 32 * i] = g[i];
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->table[buf]));
    }
  } else {
    // ------------------------------------------------------------------ MMA issuer (the pair's leader only)
    // The whole warp walks the loop and waits on the barriers, one elected lane issues: loop state that is the same
    // in every lane stays in uniform registers, which the tcgen05 instructions take their operands from (a loop
    // inside "if (lane == 0)" pays a register-to-uniform move per operand per instruction).
    if (rank == 0) {
      int tl = 0;
      bool ok = true;
      int s = 0;
      uint32_t phase = 0;
      const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
      const uint64_t ad0 = umma_desc_sw128(ring_u32), bd0 = umma_desc_sw128(ring_u32 + A_BYTES);
      constexpr uint64_t STAGE_UNITS = STAGE_BYTES >> 4;  // descriptor start addresses count 16-byte units
      uint64_t ad = ad0, bd = bd0;
      int half_next = unit < total_items ? p.mtiles[unit / NT].w : 0;
      PROF_DECL(7)
      PROF_T(m_start)
      for (int item = unit; item < total_items && ok; item += units, ++tl) {
        const int half = half_next;
        if (item + units < total_items) half_next = p.mtiles[(item + units) / NT].w;  // needed one item from now
        const uint32_t idesc = umma_idesc_f16(ITEM_N, half ? TOK_ROWS : 2 * TOK_ROWS);
        const int buf = tl & 1;
        PROF_T(m0)
        if (!mbar_wait(smem_u32(&sh->tmem_empty[buf]), ((tl >> 1) & 1) ^ 1, abort_flag)) break;
        PROF_T(m1)
        PROF_ADD(4, m0, m1)
        tc_fence_after();
        const uint32_t d = tmem_base + (uint32_t)(buf * ITEM_N);
        for (int kb = 0; kb < KB; ++kb) {
          PROF_T(k0)
          if (!mbar_wait(full0 + 8 * s, phase, abort_flag)) {
            ok = false;
            break;
          }
          PROF_T(k2)
          tc_fence_after();
          if (elect_one()) {
            tc_mma_f16_pair(d, ad, bd, idesc, kb != 0);
            tc_mma_f16_pair(d, ad + 2, bd + 2, idesc, 1);
            tc_mma_f16_pair(d, ad + 4, bd + 4, idesc, 1);
            tc_mma_f16_pair(d, ad + 6, bd + 6, idesc, 1);
            tc_commit_pair(empty0 + 8 * s, 3);
          }
          __syncwarp();
          PROF_T(k4)
          PROF_ADD(0, k0, k2) PROF_ADD(2, k2, k4) PROF_ADD(5, 0, 1)
          if (++s == ST) {
            s = 0;
            phase ^= 1;
            ad = ad0;
            bd = bd0;
          } else {
            ad += STAGE_UNITS;
            bd += STAGE_UNITS;
          }
        }
        if (ok && elect_one()) tc_commit_pair(smem_u32(&sh->tmem_full[buf]), 3);
        __syncwarp();
      }
      PROF_T(m_end)
      PROF_ADD(6, m_start, m_end)
      if (lane == 0) { PROF_OUT(8, 7) }
    }
    __syncwarp();
   }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && sh->abort_flag) atomicExch(p.status, 11 + MODE);
  cluster_sync_all();  // neither CTA frees its TMEM or leaves while the other may still use its memory
  if (warp == R::MMA) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
  }
#ifdef B200MOE_GG_PROFILE
  if (tid == 0 && blockIdx.x < 160) g_gg_pairs[MODE][1][blockIdx.x] = gtimer();
  if (tid == 0 && blockIdx.x == 0) g_gg_prof[MODE][31] = clock64() - clk_start;
#endif
}

// Token-tile list of the grouped GEMM: {slot, first sorted position, rows <= 256, half}.  half = 1: at most 128
// rows, run as M = 128 over the pair.  Full tiles first, then the 129..255-row tiles, then the half tiles, so that
// the static round-robin hands every CTA pair a similar mix.
__global__ void __launch_bounds__(1024) build_ttiles_kernel(const int32_t* __restrict__ offsets, int num_slots,
                                                            int4* __restrict__ tiles, int32_t* __restrict__ num_tiles,
                                                            int32_t* __restrict__ pad_off) {
  // thread e: expert e (num_slots <= 1024).  Exclusive scans of the three tile counts over the experts: warp
  // shuffles, then the warp totals.  A fourth scan gives pad_off[e]: how far expert e's rows are shifted in the
  // per-route output of the down GEMM, where every expert's segment is padded to a multiple of 32 rows (so that any
  // 32 consecutive tile rows can be written as one box).
  constexpr int NC = 4;
  __shared__ int32_t wtot[NC][32];
  const int e = threadIdx.x, lane = e & 31, warp = e >> 5;
  int begin = 0, cnt = 0;
  if (e < num_slots) {
    begin = offsets[e];
    cnt = offsets[e + 1] - begin;
  }
  const int rem = cnt % TN;
  const int n[NC] = {cnt / TN, rem > TN / 2 ? 1 : 0, (rem > 0 && rem <= TN / 2) ? 1 : 0, (32 - (cnt & 31)) & 31};
  int sc[NC] = {n[0], n[1], n[2], n[3]};  // inclusive scans inside the warp
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
#pragma unroll
    for (int c = 0; c < NC; ++c) {
      const int a = __shfl_up_sync(0xffffffffu, sc[c], o);
      if (lane >= o) sc[c] += a;
    }
  }
  if (lane == 31)
    for (int c = 0; c < NC; ++c) wtot[c][warp] = sc[c];
  __syncthreads();
  int before[NC] = {0, 0, 0, 0}, total[NC] = {0, 0, 0, 0};
  for (int w = 0; w < 32; ++w)
    for (int c = 0; c < NC; ++c) {
      if (w < warp) before[c] += wtot[c][w];
      total[c] += wtot[c][w];
    }
  if (e == 0) *num_tiles = total[0] + total[1] + total[2];
  if (e < num_slots) {
    int o = before[0] + sc[0] - n[0];
    for (int i = 0; i < n[0]; ++i, ++o) tiles[o] = make_int4(e, begin + i * TN, TN, 0);
    if (n[1]) tiles[total[0] + before[1] + sc[1] - 1] = make_int4(e, begin + cnt - rem, rem, 0);
    if (n[2]) tiles[total[0] + total[1] + before[2] + sc[2] - 1] = make_int4(e, begin + cnt - rem, rem, 1);
    pad_off[e] = before[3] + sc[3] - n[3];
  }
}

// Token rows in expert order for the gate_up GEMM: xs[pos] = fp16(x[token of the route at sorted position pos] *
// 2^s), s chosen per row so that the largest element lands just under the fp16 range (exact for bf16 inputs unless
// an element is 2^28 below the row maximum), inv[pos] = 2^-s.  One warp per row; the rows may live on another GPU
// (expert parallel: `src_peers` holds every rank's token buffer, peer-mapped; plain loads).
__global__ void __launch_bounds__(256) gather_rows_f16_kernel(const __nv_bfloat16* __restrict__ x, int64_t lda,
                                                              const __nv_bfloat16* const* __restrict__ src_peers,
                                                              int tokens_per_rank, const int32_t* __restrict__ sorted_routes,
                                                              const int32_t* __restrict__ offsets, int num_slots, int top_k,
                                                              int H, __half* __restrict__ xs, float* __restrict__ inv_out,
                                                              const float* __restrict__ topk_w, float* __restrict__ w_sorted) {
  const int lane = threadIdx.x & 31;
  const int64_t pos = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (pos >= offsets[num_slots]) return;
  const int token = sorted_routes[pos] / top_k;
  if (lane == 0) w_sorted[pos] = topk_w[sorted_routes[pos]];
  const __nv_bfloat16* row;
  if (src_peers != nullptr) row = src_peers[token / tokens_per_rank] + (int64_t)(token % tokens_per_rank) * lda;
  else row = x + (int64_t)token * lda;
  __half* dst = xs + pos * H;
  // every token row is read top_k times, far apart in time, while 8 T rows stream out: keep the reads in L2
  const uint64_t keep = l2_policy_keep(), stream = l2_policy_stream();
  const bool local = src_peers == nullptr;
  // rows up to 2048 elements stay in registers between the two passes; longer rows are read twice
  uint4 v[8];
  float amax = 0.f;
  for (int k0 = 0; k0 < H; k0 += 2048) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = k0 + (i * 32 + lane) * 8;
      v[i] = make_uint4(0, 0, 0, 0);
      if (k < H) v[i] = local ? ldg_nc_v4_policy(row + k, keep) : ldg_nc_v4(row + k);
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        amax = fmaxf(amax, fabsf(bf16_bits_to_float(w[c] & 0xffffu)));
        amax = fmaxf(amax, fabsf(__uint_as_float(w[c] & 0xffff0000u)));
      }
    }
  }
  amax = warp_max(amax);
  float scale, inv;
  f16_row_scale(amax, scale, inv);
  if (lane == 0) inv_out[pos] = inv;
  for (int k0 = 0; k0 < H; k0 += 2048) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = k0 + (i * 32 + lane) * 8;
      if (k >= H) continue;
      if (H > 2048) v[i] = local ? ldg_nc_v4_policy(row + k, keep) : ldg_nc_v4(row + k);
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
      uint32_t o[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const __half2 h = __floats2half2_rn(bf16_bits_to_float(w[c] & 0xffffu) * scale, __uint_as_float(w[c] & 0xffff0000u) * scale);
        o[c] = *reinterpret_cast<const uint32_t*>(&h);
      }
      stg_v4_policy(dst + k, make_uint4(o[0], o[1], o[2], o[3]), stream);
    }
  }
}

// The same copy written the other way round: one warp per TOKEN reads the row once, scales and converts it in
// registers and writes it to the sorted position of each of its routes (inv_routes: route -> position, -1 = no expert
// here).  Reads T rows instead of top_k x T; the writes are the same.  Rows of up to 2048 elements.
__global__ void __launch_bounds__(256) scatter_rows_f16_kernel(const __nv_bfloat16* __restrict__ x, int64_t lda, int T,
                                                               const int32_t* __restrict__ inv_routes, int top_k, int H,
                                                               __half* __restrict__ xs, float* __restrict__ inv_out,
                                                               const float* __restrict__ topk_w,
                                                               float* __restrict__ w_sorted) {
  const int lane = threadIdx.x & 31;
  const int64_t t = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  int my_pos = lane < top_k ? inv_routes[t * top_k + lane] : -1;   // lane k holds the position of route k
  if (my_pos >= 0) w_sorted[my_pos] = topk_w[t * top_k + lane];     // router weights in sorted order, for the down GEMM
  if (__ballot_sync(0xffffffffu, my_pos >= 0) == 0u) return;         // none of the token's experts lives here
  const __nv_bfloat16* row = x + t * lda;
  const uint64_t stream = l2_policy_stream();
  uint4 v[8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int k = (i * 32 + lane) * 8;
    v[i] = make_uint4(0, 0, 0, 0);
    if (k < H) v[i] = ldg_nc_v4(row + k);
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      amax = fmaxf(amax, fabsf(bf16_bits_to_float(w[c] & 0xffffu)));
      amax = fmaxf(amax, fabsf(__uint_as_float(w[c] & 0xffff0000u)));
    }
  }
  amax = warp_max(amax);
  float scale, inv;
  f16_row_scale(amax, scale, inv);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
    uint32_t o[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const __half2 h = __floats2half2_rn(bf16_bits_to_float(w[c] & 0xffffu) * scale, __uint_as_float(w[c] & 0xffff0000u) * scale);
      o[c] = *reinterpret_cast<const uint32_t*>(&h);
    }
    v[i] = make_uint4(o[0], o[1], o[2], o[3]);
  }
  for (int kk = 0; kk < top_k; ++kk) {
    const int pos = __shfl_sync(0xffffffffu, my_pos, kk);
    if (pos < 0) continue;
    __half* dst = xs + (int64_t)pos * H;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int k = (i * 32 + lane) * 8;
      if (k < H) stg_v4_policy(dst + k, v[i], stream);
    }
    if (lane == 0) inv_out[pos] = inv;
  }
}

// out[t] = bf16(sum_k f32(ic3[t,k])) in k order; optional merge with the shared expert.
template <int TOPK>
__global__ void __launch_bounds__(256) combine_kernel(const __nv_bfloat16* __restrict__ ic3,
                                                      const int32_t* __restrict__ inv,  // route -> sorted position (-1: none) or null
                                                      const int32_t* __restrict__ pad_off,  // with inv: row = position + pad_off[id]
                                                      const int32_t* __restrict__ ids, int num_slots, int T,
                                                      int top_k, int H, const __nv_bfloat16* __restrict__ shared,
                                                      const __nv_bfloat16* __restrict__ gate,
                                                      __nv_bfloat16* __restrict__ out) {
  // TOPK > 0: the route count is known at compile time, so all ids and then all rows are requested before the
  // first add (one memory round trip per thread instead of one per route); TOPK == 0: any top_k, route by route.
  const int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // one 8-column group
  const int hv = H >> 3;
  if (v >= (int64_t)T * hv) return;
  const int t = (int)(v / hv), h = (int)(v - (int64_t)t * hv) * 8;
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  auto add = [&](const uint4& q) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[2 * j] += bf16_bits_to_float(w[j] & 0xffffu);
      acc[2 * j + 1] += __uint_as_float(w[j] & 0xffff0000u);
    }
  };
  if (TOPK > 0) {
    bool live[TOPK > 0 ? TOPK : 1];
    int64_t row[TOPK > 0 ? TOPK : 1];
    uint4 q[TOPK > 0 ? TOPK : 1];
#pragma unroll
    for (int k = 0; k < TOPK; ++k) {
      live[k] = true;
      row[k] = (int64_t)t * TOPK + k;
      if (inv != nullptr) {   // rows in sorted order: the permutation's inverse says where (and whether) a route landed
        const int pos = inv[(int64_t)t * TOPK + k];
        live[k] = pos >= 0;
        row[k] = live[k] ? pos + pad_off[ids[(int64_t)t * TOPK + k]] : 0;
      } else if (ids != nullptr) {
        const int id = ids[(int64_t)t * TOPK + k];
        live[k] = id >= 0 && id < num_slots;  // dropped route: its ic3 row was never written
      }
    }
#pragma unroll
    for (int k = 0; k < TOPK; ++k) {
      q[k] = make_uint4(0, 0, 0, 0);
      if (live[k]) q[k] = ldg_nc_v4(ic3 + row[k] * H + h);
    }
#pragma unroll
    for (int k = 0; k < TOPK; ++k)
      if (live[k]) add(q[k]);
  } else {
    for (int k = 0; k < top_k; ++k) {
      int64_t row = (int64_t)t * top_k + k;
      if (inv != nullptr) {
        const int pos = inv[row];
        if (pos < 0) continue;
        row = pos + pad_off[ids[row]];
      } else if (ids != nullptr) {
        const int id = ids[row];
        if (id < 0 || id >= num_slots) continue;
      }
      add(*reinterpret_cast<const uint4*>(ic3 + row * H + h));
    }
  }
  if (shared != nullptr) {
    const float gl = __bfloat162float(gate[t]);
    const float sig = bf16_round(1.0f / (1.0f + expf(-gl)));
    const uint4 q = *reinterpret_cast<const uint4*>(shared + (int64_t)t * H + h);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[2 * j] = bf16_round(acc[2 * j]) + bf16_round(bf16_bits_to_float(w[j] & 0xffffu) * sig);
      acc[2 * j + 1] = bf16_round(acc[2 * j + 1]) + bf16_round(__uint_as_float(w[j] & 0xffff0000u) * sig);
    }
  }
  *reinterpret_cast<uint4*>(out + (int64_t)t * H + h) =
      make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
}

static int launch_combine(const __nv_bfloat16* ic3, const int32_t* inv, const int32_t* pad_off, const int32_t* ids,
                          int num_slots, int T, int top_k, int H, const __nv_bfloat16* shared, const __nv_bfloat16* gate, __nv_bfloat16* out, cudaStream_t st) {
  const int64_t groups = (int64_t)T * (H / 8);
  const unsigned grid = (unsigned)((groups + 255) / 256);
  if (top_k == 8) combine_kernel<8><<<grid, 256, 0, st>>>(ic3, inv, pad_off, ids, num_slots, T, top_k, H, shared, gate, out);
  else if (top_k == 1) combine_kernel<1><<<grid, 256, 0, st>>>(ic3, inv, pad_off, ids, num_slots, T, top_k, H, shared, gate, out);
  else combine_kernel<0><<<grid, 256, 0, st>>>(ic3, inv, pad_off, ids, num_slots, T, top_k, H, shared, gate, out);
  return check_launch();
}

// 8 outputs per thread: two 16-byte loads, one 16-byte store
__global__ void __launch_bounds__(256) silu_and_mul_v8_kernel(const __nv_bfloat16* __restrict__ in,
                                                              __nv_bfloat16* __restrict__ out, int64_t rows, int D) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int dv = D >> 3;
  if (i >= rows * dv) return;
  const int64_t r = i / dv;
  const int d = (int)(i - r * dv) * 8;
  const uint4 g = ldg_nc_v4(in + r * 2 * D + d), u = ldg_nc_v4(in + r * 2 * D + D + d);
  const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j)
    o[j] = pack_bf16x2(silu_mul(bf16_bits_to_float(gw[j] & 0xffffu), bf16_bits_to_float(uw[j] & 0xffffu)),
                       silu_mul(__uint_as_float(gw[j] & 0xffff0000u), __uint_as_float(uw[j] & 0xffff0000u)));
  *reinterpret_cast<uint4*>(out + r * D + d) = make_uint4(o[0], o[1], o[2], o[3]);
}

__global__ void silu_and_mul_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t rows, int D) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * D) return;
  const int64_t r = i / D;
  const int d = (int)(i - r * D);
  out[i] = __float2bfloat16_rn(silu_mul(__bfloat162float(in[r * 2 * D + d]), __bfloat162float(in[r * 2 * D + D + d])));
}


struct PrefillWs {
  void* perm_ws;
  int64_t perm_bytes;
  int32_t *sorted_routes, *inv_routes, *offsets, *num_mtiles, *pad_off;
  int4* mtiles;
  __half *xs, *ic2;
  float *a_inv, *w_sorted;
  __nv_bfloat16* ic3;
  int64_t bytes;
};
static PrefillWs carve_prefill_ws(void* ws, int T, int top_k, int H, int I, int slots) {
  PrefillWs w;
  auto up = [](int64_t v) { return (v + 1023) / 1024 * 1024; };
  char* p = reinterpret_cast<char*>(ws);
  const int64_t R = (int64_t)T * top_k;
  int64_t off = 0;
  w.perm_bytes = b200moe_permute_workspace_bytes((int)R, slots);
  w.perm_ws = p + off; off += up(w.perm_bytes);
  w.sorted_routes = reinterpret_cast<int32_t*>(p + off); off += up(R * 4);
  w.inv_routes = reinterpret_cast<int32_t*>(p + off); off += up(R * 4);
  w.offsets = reinterpret_cast<int32_t*>(p + off); off += up(((int64_t)slots + 2) * 4);
  w.num_mtiles = reinterpret_cast<int32_t*>(p + off); off += up(16);
  w.pad_off = reinterpret_cast<int32_t*>(p + off); off += up(((int64_t)slots + 1) * 4);
  w.mtiles = reinterpret_cast<int4*>(p + off); off += up((R / TN + slots + 2) * 16);
  w.a_inv = reinterpret_cast<float*>(p + off); off += up((R + TN) * 4);
  w.w_sorted = reinterpret_cast<float*>(p + off); off += up((R + TN) * 4);
  w.xs = reinterpret_cast<__half*>(p + off); off += up((R + TN) * H * 2);
  w.ic2 = reinterpret_cast<__half*>(p + off); off += up((R + TN) * I * 2);
  w.ic3 = reinterpret_cast<__nv_bfloat16*>(p + off); off += up((R + 32 * (int64_t)slots) * H * 2);  // segments padded to 32 rows
  w.bytes = off;
  return w;
}

// Tensor map of a row-major fp16 matrix [rows, cols] (row pitch in elements): boxes of 64 columns x 64 rows,
// 128-byte swizzle.  The encoder lives in the driver; it is looked up once.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static std::mutex g_prefill_lock;
static EncodeTiledFn g_encode_tiled = nullptr;
static int encode_rows_map(CUtensorMap* map, const void* base, int64_t rows, int64_t cols, int64_t pitch,
                           int box_rows = 64, CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_FLOAT16, int box_cols = BK,
                           CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn& encode = g_encode_tiled;
  {
    std::lock_guard<std::mutex> guard(g_prefill_lock);
    if (!encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
      if (e != cudaSuccess) return (int)e;
      if (!fn || q != cudaDriverEntryPointSuccess) return B200MOE_E_DEVICE;
      encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
  }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)pitch * 2};
  const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows}, elem[2] = {1, 1};
  const CUresult r = encode(map, dtype, 2, const_cast<void*>(base), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : B200MOE_E_ALIGN;
}

// Tensor map of a bank role seen as bytes [slots, rows, row_bytes] (row pitch = row_bytes, slot pitch given):
// boxes of box_bytes x 64 rows x 1 slot.
static int encode_bank_map(CUtensorMap* map, const void* base, int64_t slots, int64_t rows, int64_t row_bytes,
                           int64_t slot_pitch, int box_bytes, bool swizzle128) {
  CUtensorMap probe;
  if (int rc = encode_rows_map(&probe, base, 64, 64, 64)) {  // makes sure the encoder has been looked up
    if (rc != B200MOE_E_ALIGN) return rc;
  }
  const cuuint64_t dims[3] = {(cuuint64_t)row_bytes, (cuuint64_t)rows, (cuuint64_t)slots};
  const cuuint64_t strides[2] = {(cuuint64_t)row_bytes, (cuuint64_t)slot_pitch};
  const cuuint32_t box[3] = {(cuuint32_t)box_bytes, 64, 1}, elem[3] = {1, 1, 1};
  const CUresult r = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                                    swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : B200MOE_E_ALIGN;
}

}  // namespace b200moe

using namespace b200moe;

#ifdef B200MOE_GG_PROFILE
extern "C" int b200moe_debug_gg_pairs(unsigned long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_gg_pairs, sizeof(unsigned long long) * 2 * 2 * 160);
}
extern "C" int b200moe_debug_gg_profile(long long* host_out) {
  return (int)cudaMemcpyFromSymbol(host_out, g_gg_prof, sizeof(long long) * 2 * 32);
}
#endif

extern "C" int64_t b200moe_prefill_workspace_bytes(int T, int top_k, int hidden, int intermediate, int num_slots) {
  if (T < 0 || top_k < 1 || num_slots < 1) return 0;
  return carve_prefill_ws(nullptr, T, top_k, hidden, intermediate, num_slots).bytes;
}

// One grouped GEMM launch: `units` clusters of two CTAs.
template <int MODE>
static int launch_grouped_gemm(const GgParams& g, int units, cudaStream_t st) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * units);
  cfg.blockDim = dim3(Roles<MODE>::THREADS);
  cfg.dynamicSmemBytes = GG_SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<MODE>, g);
  return e == cudaSuccess ? 0 : (int)e;
}

// How many CTA pairs of the grouped GEMM can be resident at once.
template <int MODE>
static int resident_pairs(int sm_count) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * (sm_count / 2));
  cfg.blockDim = dim3(Roles<MODE>::THREADS);
  cfg.dynamicSmemBytes = GG_SMEM;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, grouped_gemm_kernel<MODE>, &cfg) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return n;
}

// Launch state that belongs to a device (function attributes and the occupancy result are per device): looked up
// once per device ordinal under a lock.
struct PrefillDevice {
  bool ready = false;
  int pairs = 0;
};
static PrefillDevice g_prefill_dev[64];

static int prefill_device_state(int* pairs) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return B200MOE_E_DEVICE;
  std::lock_guard<std::mutex> guard(g_prefill_lock);
  PrefillDevice& d = g_prefill_dev[dev];
  if (!d.ready) {
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess) return (int)e;
    if (prop.major != 10) return B200MOE_E_DEVICE;
    e = cudaFuncSetAttribute(grouped_gemm_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GG_SMEM);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(grouped_gemm_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)GG_SMEM);
    if (e != cudaSuccess) return (int)e;
    d.pairs = std::min(resident_pairs<0>(prop.multiProcessorCount), resident_pairs<1>(prop.multiProcessorCount));
    if (d.pairs < 1) return B200MOE_E_DEVICE;
    d.ready = true;
  }
  *pairs = d.pairs;
  return 0;
}

static int prefill_stages_impl(const void* x, const b200moe_banks* banks, const float* topk_weights,
                               const int32_t* topk_ids, int T, int top_k, const void* shared,
                               const void* shared_gate_logit, void* out, void* workspace, int64_t workspace_bytes,
                               int32_t* status, int stage_mask, void* const* out_peers, int routes_per_rank,
                               int64_t route_offset, int64_t total_routes, void* stream) {
  if (T == 0) return 0;
  if (!banks || !banks->gate_up || !banks->gate_up_scale || !banks->gate_up_global || !banks->down ||
      !banks->down_scale || !banks->down_global || !x || !topk_weights || !topk_ids || !out || !workspace || !status)
    return B200MOE_E_NULL;
  const int H = banks->hidden, I = banks->intermediate, S = banks->num_slots;
  // an item is 256 weight rows: 128 gate + 128 up rows of gate_up, 256 rows of down; stages are 64 k wide
  if (T < 0 || top_k < 1 || S < 1 || S > 1024 || H % ITEM_N || I % (ITEM_N / 2) || H % BK || I % BK ||
      (int64_t)T * top_k > (1ll << 30))
    return B200MOE_E_SHAPE;
  if ((shared == nullptr) != (shared_gate_logit == nullptr)) return B200MOE_E_NULL;
  if (!aligned16(x) || !aligned16(out) || !aligned16(workspace) || !aligned16(banks->gate_up) ||
      !aligned16(banks->down) || !aligned16(banks->gate_up_scale) || !aligned16(banks->down_scale) || (reinterpret_cast<uintptr_t>(banks->gate_up_global) & 15) ||
      (reinterpret_cast<uintptr_t>(banks->down_global) & 15) || (shared && !aligned16(shared)))
    return B200MOE_E_ALIGN;
  PrefillWs ws = carve_prefill_ws(workspace, T, top_k, H, I, S);
  if (workspace_bytes < ws.bytes) return B200MOE_E_WORKSPACE;
  b200moe_banks nb;
  {
    const int nrc = normalize_banks(banks, &nb);
    if (nrc) return nrc;
    banks = &nb;
  }
  // the epilogue reads the per-row globals as 16-byte vectors
  if ((banks->slot_stride[2] & 15) || (banks->slot_stride[5] & 15)) return B200MOE_E_ALIGN;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int R = T * top_k;
  int pairs = 0;
  int rc = prefill_device_state(&pairs);
  if (rc) return rc;

  if (stage_mask & B200MOE_STAGE_PLAN) {
    cudaError_t ce = cudaMemsetAsync(status, 0, 4 * sizeof(int32_t), st);
    if (ce != cudaSuccess) return (int)ce;
    // rows that fit a warp's registers are read once per token and written to each route's position; longer rows (or
    // more routes per token than a warp has lanes) are fetched per sorted position
    const bool by_token = H <= 2048 && top_k <= 32;
    rc = permute_with_inverse(topk_ids, R, S, 1, nullptr, 0, nullptr, 0, nullptr, ws.sorted_routes, ws.offsets,
                              ws.inv_routes, ws.perm_ws, ws.perm_bytes, stream);
    if (rc) return rc;
    build_ttiles_kernel<<<1, 1024, 0, st>>>(ws.offsets, S, ws.mtiles, ws.num_mtiles, ws.pad_off);
    if ((rc = check_launch())) return rc;
    if (by_token)
      scatter_rows_f16_kernel<<<(unsigned)(((int64_t)T * 32 + 255) / 256), 256, 0, st>>>(
          reinterpret_cast<const __nv_bfloat16*>(x), H, T, ws.inv_routes, top_k, H, ws.xs, ws.a_inv, topk_weights, ws.w_sorted);
    else
      gather_rows_f16_kernel<<<(unsigned)(((int64_t)R * 32 + 255) / 256), 256, 0, st>>>(
          reinterpret_cast<const __nv_bfloat16*>(x), H, nullptr, 1, ws.sorted_routes, ws.offsets, S, top_k, H, ws.xs, ws.a_inv,
          topk_weights, ws.w_sorted);
    if ((rc = check_launch())) return rc;
  }

  const int max_mtiles = R / TN + S;  // token tiles: full ones plus at most one partial per slot
  GgParams g1{};
  if ((rc = encode_rows_map(&g1.a_map, ws.xs, (int64_t)R + TN, H, H))) return rc;
  const bool staged1 = H % (SUPER * BK) == 0, staged2 = I % (SUPER * BK) == 0;
  if (staged1) {
    if ((rc = encode_bank_map(&g1.w_map, banks->gate_up, S, 2 * I, H / 2, banks->slot_stride[0], SUPER * BK / 2, true))) return rc;
    if ((rc = encode_bank_map(&g1.s_map, banks->gate_up_scale, S, 2 * I, H / 16, banks->slot_stride[1], SUPER * BK / 16, false))) return rc;
  }
  g1.w_staged = staged1;
  g1.packed = banks->gate_up;
  g1.scales = banks->gate_up_scale;
  g1.globals = banks->gate_up_global;
  g1.packed_stride = banks->slot_stride[0];
  g1.scale_stride = banks->slot_stride[1];
  g1.global_stride = banks->slot_stride[2];
  g1.N = 2 * I;
  g1.K = H;
  g1.NT = I / (ITEM_N / 2);
  g1.half_n = I;
  g1.mtiles = ws.mtiles;
  g1.num_mtiles = ws.num_mtiles;
  g1.sorted_routes = ws.sorted_routes;
  g1.topk_w = topk_weights;
  g1.a_inv = ws.a_inv;
  g1.w_sorted = ws.w_sorted;
  g1.out = ws.ic2;
  g1.status = status;
  if (stage_mask & B200MOE_STAGE_GEMM1) {
    rc = launch_grouped_gemm<0>(g1, (int)std::min<int64_t>(pairs, (int64_t)max_mtiles * g1.NT), st);
    if (rc) return rc;
  }

  GgParams g2 = g1;
  if ((rc = encode_rows_map(&g2.a_map, ws.ic2, (int64_t)R + TN, I, I))) return rc;
  if (staged2) {
    if ((rc = encode_bank_map(&g2.w_map, banks->down, S, H, I / 2, banks->slot_stride[3], SUPER * BK / 2, true))) return rc;
    if ((rc = encode_bank_map(&g2.s_map, banks->down_scale, S, H, I / 16, banks->slot_stride[4], SUPER * BK / 16, false))) return rc;
  }
  g2.w_staged = staged2;
  g2.packed = banks->down;
  g2.scales = banks->down_scale;
  g2.globals = banks->down_global;
  g2.packed_stride = banks->slot_stride[3];
  g2.scale_stride = banks->slot_stride[4];
  g2.global_stride = banks->slot_stride[5];
  g2.N = H;
  g2.K = I;
  g2.NT = H / ITEM_N;
  g2.a_inv = nullptr;
  g2.out = ws.ic3;
  g2.out_peers = reinterpret_cast<__nv_bfloat16* const*>(out_peers);
  g2.routes_per_rank = routes_per_rank > 0 ? routes_per_rank : 1;
  g2.route_offset = route_offset;
  g2.total_routes = total_routes > 0 ? total_routes : (int64_t)1 << 62;
  // Per-route rows: in sorted (expert) order when they stay in this workspace for the combine stage -- a tile's rows
  // are then consecutive and leave by TMA store, and the combine stage finds them through the inverse permutation;
  // in route order when they go to their home GPUs or when the caller reads them (B200MOE_STAGE_ROUTE_ORDER).
  const bool sorted_out = out_peers == nullptr && !(stage_mask & B200MOE_STAGE_ROUTE_ORDER);
  g2.out_sorted = sorted_out;
  g2.pad_off = ws.pad_off;
  if (sorted_out && (rc = encode_rows_map(&g2.o_map, ws.ic3, (int64_t)R + 32 * (int64_t)S, H, H, 32, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 32, CU_TENSOR_MAP_SWIZZLE_64B))) return rc;
  if (stage_mask & B200MOE_STAGE_GEMM2) {
    rc = launch_grouped_gemm<1>(g2, (int)std::min<int64_t>(pairs, (int64_t)max_mtiles * g2.NT), st);
    if (rc) return rc;
  }
  if (stage_mask & B200MOE_STAGE_COMBINE) {
    rc = launch_combine(ws.ic3, sorted_out ? ws.inv_routes : nullptr, ws.pad_off, topk_ids, S, T, top_k, H,
                        reinterpret_cast<const __nv_bfloat16*>(shared),
                        reinterpret_cast<const __nv_bfloat16*>(shared_gate_logit), reinterpret_cast<__nv_bfloat16*>(out), st);
    if (rc) return rc;
  }
  return 0;
}

extern "C" int b200moe_prefill_stages(const void* x, const b200moe_banks* banks, const float* topk_weights,
                                      const int32_t* topk_ids, int T, int top_k, const void* shared,
                                      const void* shared_gate_logit, void* out, void* workspace,
                                      int64_t workspace_bytes, int32_t* status, int stage_mask, void* stream) {
  return prefill_stages_impl(x, banks, topk_weights, topk_ids, T, top_k, shared, shared_gate_logit, out, workspace,
                             workspace_bytes, status, stage_mask, nullptr, 0, 0, 0, stream);
}

extern "C" int b200moe_prefill_ep_routes(const void* x, const b200moe_banks* local_banks, const float* weights,
                                         const int32_t* local_ids, int T, int first_token, int top_k,
                                         void* const* peer_ic3, int world, int tokens_per_rank, void* workspace,
                                         int64_t workspace_bytes, int32_t* status, void* stream) {
  if (!peer_ic3) return B200MOE_E_NULL;
  // the T tokens are the box's tokens first_token, first_token + 1, ... modulo world * tokens_per_rank
  if (world < 1 || tokens_per_rank < 1 || first_token < 0 || T < 0 ||
      (int64_t)first_token >= (int64_t)world * tokens_per_rank || (int64_t)T > (int64_t)world * tokens_per_rank)
    return B200MOE_E_SHAPE;
  return prefill_stages_impl(x, local_banks, weights, local_ids, T, top_k, nullptr, nullptr, const_cast<void*>(x),
                             workspace, workspace_bytes, status,
                             B200MOE_STAGE_PLAN | B200MOE_STAGE_GEMM1 | B200MOE_STAGE_GEMM2, peer_ic3,
                             tokens_per_rank * top_k, (int64_t)first_token * top_k,
                             (int64_t)world * tokens_per_rank * top_k, stream);
}

extern "C" int b200moe_prefill_experts(const void* x, const b200moe_banks* banks, const float* topk_weights,
                                       const int32_t* topk_ids, int T, int top_k, const void* shared,
                                       const void* shared_gate_logit, void* out, void* workspace,
                                       int64_t workspace_bytes, int32_t* status, void* stream) {
  return b200moe_prefill_stages(x, banks, topk_weights, topk_ids, T, top_k, shared, shared_gate_logit, out, workspace,
                                workspace_bytes, status, B200MOE_STAGE_ALL, stream);
}

extern "C" int b200moe_silu_and_mul(const void* in, void* out, int rows, int D, void* stream) {
  if (rows == 0) return 0;
  if (!in || !out) return B200MOE_E_NULL;
  if (rows < 0 || D < 1) return B200MOE_E_SHAPE;
  const int64_t n = (int64_t)rows * D;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (D % 8 == 0 && aligned16(in) && aligned16(out))
    silu_and_mul_v8_kernel<<<(unsigned)((n / 8 + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), rows, D);
  else
    silu_and_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const __nv_bfloat16*>(in), reinterpret_cast<__nv_bfloat16*>(out), rows, D);
  return check_launch();
}

extern "C" int b200moe_shared_epilogue(const void* routed, const void* shared, const void* gate, void* out, int T, int H,
                                       void* stream) {
  if (T == 0) return 0;
  if (!routed || !shared || !gate || !out) return B200MOE_E_NULL;
  if (T < 0 || H < 8 || H % 8) return B200MOE_E_SHAPE;
  if (!aligned16(routed) || !aligned16(shared) || !aligned16(out)) return B200MOE_E_ALIGN;
  return launch_combine(reinterpret_cast<const __nv_bfloat16*>(routed), nullptr, nullptr, nullptr, 0, T, 1, H,
                        reinterpret_cast<const __nv_bfloat16*>(shared), reinterpret_cast<const __nv_bfloat16*>(gate),
                        reinterpret_cast<__nv_bfloat16*>(out), reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_sum_routes(const void* in, void* out, int T, int top_k, int H, void* stream) {
  if (T == 0) return 0;
  if (!in || !out) return B200MOE_E_NULL;
  if (T < 0 || top_k < 1 || H < 8 || H % 8) return B200MOE_E_SHAPE;
  if (!aligned16(in) || !aligned16(out)) return B200MOE_E_ALIGN;
  return launch_combine(reinterpret_cast<const __nv_bfloat16*>(in), nullptr, nullptr, nullptr, 0, T, top_k, H, nullptr, nullptr,
                        reinterpret_cast<__nv_bfloat16*>(out), reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int b200moe_combine_routes(const void* ic3, const int32_t* topk_ids, int num_slots, int T, int top_k, int H,
                                      const void* shared, const void* shared_gate_logit, void* out, void* stream) {
  if (T == 0) return 0;
  if (!ic3 || !out) return B200MOE_E_NULL;
  if ((shared == nullptr) != (shared_gate_logit == nullptr)) return B200MOE_E_NULL;
  if (T < 0 || top_k < 1 || H < 8 || H % 8) return B200MOE_E_SHAPE;
  if (!aligned16(ic3) || !aligned16(out) || (shared && !aligned16(shared))) return B200MOE_E_ALIGN;
  return launch_combine(reinterpret_cast<const __nv_bfloat16*>(ic3), nullptr, nullptr, topk_ids, num_slots, T, top_k, H,
                        reinterpret_cast<const __nv_bfloat16*>(shared), reinterpret_cast<const __nv_bfloat16*>(shared_gate_logit),
                        reinterpret_cast<__nv_bfloat16*>(out), reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int64_t b200moe_prefill_ic3_offset(int T, int top_k, int hidden, int intermediate, int num_slots) {
  if (T < 0 || top_k < 1 || num_slots < 1) return -1;
  PrefillWs w = carve_prefill_ws(nullptr, T, top_k, hidden, intermediate, num_slots);
  return reinterpret_cast<char*>(w.ic3) - reinterpret_cast<char*>(0);
}
