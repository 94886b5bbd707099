// Dense bf16 linears of the prefill block on the tensor cores: router logits, the shared expert's gate_up (with its
// SwiGLU) and down projections (freetoken/python/freetoken/models/qwen3_5_moe/moe.py:20-36,66,86,99-106; the reference
// runs them as library GEMMs, freetoken/python/freetoken/layers/quantization/linear/unquantized.py:18-24).
//
//   out[t, n] = bf16( sum_k x[t, k] * w[n, k]  [+ bias[n]] )                          plain / bias
//   act[t, i] = bf16( silu(bf16(acc[t, i])) * bf16(acc[t, SI + i]) )                   gate_up + SwiGLU
//
// One CTA per tile of 128 tokens x 256 weight rows (tcgen05 cta_group::1, kind::f16 with bf16 operands, fp32
// accumulation in TMEM), both operands by TMA (64-row x 64-k boxes, 128-byte swizzle) through a four-slot ring;
// warp 4 issues the copies, warp 5 the MMAs (whole warp in the loop, one elected lane issues), warps 0-3 drain the
// double-buffered accumulator: a thread owns one token, four lanes transpose their pieces so that a store
// instruction writes contiguous 128-byte pieces.  For gate_up + SwiGLU a tile takes 128 gate rows and the 128 up
// rows of the same outputs, so a thread holds both halves of a pair.  Every wait is bounded.
#include <mutex>

#include "tc.cuh"

namespace b200moe {

constexpr int DK = 64, DM = 128;
constexpr int DA_BYTES = DM * DK * 2;
constexpr int EPI_WARPS = 8, DENSE_THREADS = (EPI_WARPS + 2) * 32;

// Tile width (weight rows per tile) and the depth of the operand ring it leaves room for.
template <int DN>
struct DenseCfg {
  static constexpr int B_BYTES = DN * DK * 2, STAGE_BYTES = DA_BYTES + B_BYTES;
  static constexpr int STAGES = DN == 256 ? 4 : 6;
};

struct DenseParams {
  CUtensorMap a_map, w_map;      // x [T, K] and w [N, K] bf16 as 64-column x 64-row boxes, 128B swizzle
  const float* bias;             // [N] or null
  __nv_bfloat16* out;            // [T, ldo]
  int T, N, K, ldo;
  int half;                      // SwiGLU: w = [2 half, K] (gate rows, then up rows), out = [T, half]
  int32_t* status;
};

struct alignas(16) DenseShared {
  unsigned long long full[6], empty[6], tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  int abort_flag;
};
template <int DN>
constexpr size_t dense_smem() {
  return 1024 + (size_t)DenseCfg<DN>::STAGES * DenseCfg<DN>::STAGE_BYTES + sizeof(DenseShared);
}

template <int DN, bool SWIGLU>
__global__ void __launch_bounds__(DENSE_THREADS, 1) dense_gemm_kernel(const __grid_constant__ DenseParams p) {
  using Cfg = DenseCfg<DN>;
  constexpr int STAGES = Cfg::STAGES, STAGE_BYTES = Cfg::STAGE_BYTES;
  constexpr int OUT_COLS = SWIGLU ? DN / 2 : DN;               // output columns of a tile
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* ring = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  DenseShared* sh = reinterpret_cast<DenseShared*>(ring + (size_t)STAGES * STAGE_BYTES);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t ring_u32 = smem_u32(ring);
  volatile int* abort_flag = &sh->abort_flag;
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&sh->full[s]), 1);
      mbar_init(smem_u32(&sh->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&sh->tmem_full[b]), 1);
      mbar_init(smem_u32(&sh->tmem_empty[b]), EPI_WARPS);
    }
    sh->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == EPI_WARPS + 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = sh->tmem_base;
  const int out_cols = SWIGLU ? p.half : p.N;
  const int n_tiles = (out_cols + OUT_COLS - 1) / OUT_COLS;
  const int m_tiles = (p.T + DM - 1) / DM;
  const int tiles = m_tiles * n_tiles;
  const int KB = p.K / DK;

  if (warp < EPI_WARPS) {
    // ---------------- epilogue: lane = token (TMEM lane quarter warp & 3), the two warps of a quarter split the columns
    const int jq = lane & 3, quarter = warp & 3, chalf = warp >> 2;
    constexpr int COLS_PER_WARP = OUT_COLS / 2;                // 128, 64 or 32
    constexpr int GROUP = COLS_PER_WARP >= 64 ? 64 : 32;       // columns converted per round: 4 pieces of GROUP / 4
    constexpr int PIECE = GROUP / 4;                           // 16 or 8 columns
    constexpr int NR = PIECE / 2;                              // registers of a piece
    int tl = 0;
    const bool wide_rows = (p.ldo & 15) == 0;   // every row starts on a 32-byte boundary
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++tl) {
      const int mt = tile / n_tiles, nt = tile - mt * n_tiles;
      const int buf = tl & 1;
      const int tok = mt * DM + quarter * 32 + lane;
      const int col_out0 = nt * OUT_COLS + chalf * COLS_PER_WARP;   // first output column of this warp
      char* dst = tok < p.T ? reinterpret_cast<char*>(p.out + (int64_t)tok * p.ldo + col_out0) : nullptr;
      const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->tmem_full[buf]), (tl >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const uint32_t tbase = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * DN + chalf * COLS_PER_WARP);
#pragma unroll 1
      for (int c = 0; c < COLS_PER_WARP; c += GROUP) {
        uint32_t v[GROUP / 16][16], u[SWIGLU ? GROUP / 16 : 1][16];
#pragma unroll
        for (int i = 0; i < GROUP / 16; ++i) {
          tc_ld16(tbase + c + 16 * i, v[i]);
          if (SWIGLU) tc_ld16(tbase + DN / 2 + c + 16 * i, u[i]);
        }
        tc_wait_ld();
        uint32_t blk[4][NR];
#pragma unroll
        for (int q = 0; q < GROUP / 2; ++q) {                  // output pair q of the group: columns c + 2q, c + 2q + 1
          const int i = (2 * q) / 16, e = (2 * q) % 16;
          float a = __uint_as_float(v[i][e]), b = __uint_as_float(v[i][e + 1]);
          if (SWIGLU) {
            a = silu_mul(bf16_round(a), bf16_round(__uint_as_float(u[i][e])));
            b = silu_mul(bf16_round(b), bf16_round(__uint_as_float(u[i][e + 1])));
          } else if (p.bias != nullptr) {
            const int n = col_out0 + c + 2 * q;
            a += n < p.N ? p.bias[n] : 0.f;
            b += n + 1 < p.N ? p.bias[n + 1] : 0.f;
          }
          blk[(2 * q) / PIECE][((2 * q) % PIECE) / 2] = pack_bf16x2(a, b);
        }
        quad_transpose<NR>(blk, jq);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          // blk[k] = piece jq of token k of the quad: PIECE output columns starting at c + PIECE * jq
          char* dk = reinterpret_cast<char*>(__shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)dst, (lane & ~3) + k));
          const int col = col_out0 + c + PIECE * jq;
          if (dk == nullptr) continue;
          char* d = dk + (c + PIECE * jq) * 2;
          if constexpr (NR == 8) {
            if (wide_rows && col + 16 <= out_cols) {   // 32 contiguous bytes per lane, whole sectors
              stg_v8(d, blk[k]);
              continue;
            }
          }
#pragma unroll
          for (int h = 0; h < NR / 4; ++h)
            if (col + 8 * (h + 1) <= out_cols) stg_v4(d + 16 * h, make_uint4(blk[k][4 * h], blk[k][4 * h + 1], blk[k][4 * h + 2], blk[k][4 * h + 3]));
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sh->tmem_empty[buf]));
    }
  } else if (warp == EPI_WARPS) {
    // ---------------- TMA: both operands
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x) {
        const int mt = tile / n_tiles, nt = tile - mt * n_tiles;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % STAGES;
          ok = mbar_wait(smem_u32(&sh->empty[s]), ((it / STAGES) & 1) ^ 1, abort_flag);
          if (!ok) break;
          const uint32_t sa = ring_u32 + s * STAGE_BYTES, sb = sa + DA_BYTES, bar = smem_u32(&sh->full[s]);
          mbar_arrive_expect_tx(bar, (uint32_t)STAGE_BYTES);
          for (int b = 0; b < DM / 64; ++b) tma_load_2d(sa + b * (64 * 128), &p.a_map, kb * DK, mt * DM + b * 64, bar);
#pragma unroll
          for (int b = 0; b < DN / 64; ++b) {
            // weight rows behind B rows 64 b .. 64 b + 63: plain tiles take DN consecutive rows; gate_up tiles take
            // DN / 2 gate rows, then the DN / 2 up rows of the same outputs
            int row;
            if (SWIGLU) row = (b < DN / 128 ? 0 : p.half) + nt * (DN / 2) + (b % (DN / 128)) * 64;
            else row = nt * DN + b * 64;
            tma_load_2d(sb + b * (64 * 128), &p.w_map, kb * DK, row, bar);
          }
        }
      }
    }
  } else {
    // ---------------- MMA issuer (the whole warp walks the loop; one elected lane issues)
    int tl = 0, s = 0;
    uint32_t phase = 0;
    bool ok = true;
    const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
    const uint64_t ad0 = umma_desc_sw128(ring_u32), bd0 = umma_desc_sw128(ring_u32 + DA_BYTES);
    constexpr uint64_t STAGE_UNITS = STAGE_BYTES >> 4;
    uint64_t ad = ad0, bd = bd0;
    const uint32_t idesc = umma_idesc_bf16(DN, DM);
    for (int tile = blockIdx.x; tile < tiles && ok; tile += gridDim.x, ++tl) {
      const int buf = tl & 1;
      if (!__all_sync(0xffffffffu, mbar_wait(smem_u32(&sh->tmem_empty[buf]), ((tl >> 1) & 1) ^ 1, abort_flag))) break;
      tc_fence_after();
      const uint32_t d = tmem_base + (uint32_t)(buf * DN);
      for (int kb = 0; kb < KB; ++kb) {
        if (!__all_sync(0xffffffffu, mbar_wait(full0 + 8 * s, phase, abort_flag))) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (elect_one()) {
          tc_mma_f16_cta(d, ad, bd, idesc, kb != 0);
          tc_mma_f16_cta(d, ad + 2, bd + 2, idesc, 1);
          tc_mma_f16_cta(d, ad + 4, bd + 4, idesc, 1);
          tc_mma_f16_cta(d, ad + 6, bd + 6, idesc, 1);
          tc_commit_cta(empty0 + 8 * s);
        }
        __syncwarp();
        if (++s == STAGES) {
          s = 0;
          phase ^= 1;
          ad = ad0;
          bd = bd0;
        } else {
          ad += STAGE_UNITS;
          bd += STAGE_UNITS;
        }
      }
      if (ok && elect_one()) tc_commit_cta(smem_u32(&sh->tmem_full[buf]));
      __syncwarp();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && sh->abort_flag) atomicExch(p.status, 21);
  if (warp == EPI_WARPS + 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// gate logit of the shared expert: out[t] = bf16(sum_k x[t, k] * w[k]); one warp per token
__global__ void __launch_bounds__(256) row_dot_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                                      __nv_bfloat16* __restrict__ out, int64_t T, int K) {
  const int lane = threadIdx.x & 31;
  const int64_t t = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (t >= T) return;
  float acc = 0.f;
  for (int k = lane * 8; k < K; k += 256) {
    const uint4 a = ldg_nc_v4(x + t * K + k), b = ldg_nc_keep_v4(w + k);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc += bf16_bits_to_float(aw[j] & 0xffffu) * bf16_bits_to_float(bw[j] & 0xffffu);
      acc += __uint_as_float(aw[j] & 0xffff0000u) * __uint_as_float(bw[j] & 0xffff0000u);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) out[t] = __float2bfloat16_rn(acc);
}

typedef CUresult (*EncodeTiledFnD)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static std::mutex g_dense_lock;
static EncodeTiledFnD g_dense_encode = nullptr;
static bool g_dense_attr[64];
static int g_dense_sms[64];

static int encode_bf16_rows(CUtensorMap* map, const void* base, int64_t rows, int64_t cols) {
  {
    std::lock_guard<std::mutex> guard(g_dense_lock);
    if (!g_dense_encode) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult q;
      cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
      if (e != cudaSuccess) return (int)e;
      if (!fn || q != cudaDriverEntryPointSuccess) return B200MOE_E_DEVICE;
      g_dense_encode = reinterpret_cast<EncodeTiledFnD>(fn);
    }
  }
  const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  const cuuint32_t box[2] = {(cuuint32_t)DK, 64}, elem[2] = {1, 1};
  const CUresult r = g_dense_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : B200MOE_E_ALIGN;
}

}  // namespace b200moe

using namespace b200moe;

template <int DN, bool SWIGLU>
static int launch_dense(const DenseParams& p, int sms, cudaStream_t stream) {
  constexpr int OUT_COLS = SWIGLU ? DN / 2 : DN;
  const int out_cols = SWIGLU ? p.half : p.N;
  const int tiles = ((p.T + DM - 1) / DM) * ((out_cols + OUT_COLS - 1) / OUT_COLS);
  dense_gemm_kernel<DN, SWIGLU><<<std::min(tiles, sms), DENSE_THREADS, dense_smem<DN>(), stream>>>(p);
  return check_launch();
}

extern "C" int b200moe_dense_linear(const void* x, const void* w, const float* bias, void* out, int T, int N, int K, int swiglu,
                                    int32_t* status, void* stream) {
  if (T == 0) return 0;
  if (!x || !w || !out || !status) return B200MOE_E_NULL;
  if (T < 0 || N < 1 || K < DK || K % DK || (swiglu && (N % 2 || (N / 2) % 64)) || (!swiglu && N % 8)) return B200MOE_E_SHAPE;
  if (swiglu && bias) return B200MOE_E_SHAPE;
  if (!aligned16(x) || !aligned16(w) || !aligned16(out)) return B200MOE_E_ALIGN;
  int dev = -1, sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= 64) return B200MOE_E_DEVICE;
  {
    std::lock_guard<std::mutex> guard(g_dense_lock);
    if (!g_dense_attr[dev]) {
      cudaDeviceProp prop;
      if ((e = cudaGetDeviceProperties(&prop, dev)) != cudaSuccess) return (int)e;
      if (prop.major != 10) return B200MOE_E_DEVICE;
      if ((e = cudaFuncSetAttribute(dense_gemm_kernel<256, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)dense_smem<256>())) != cudaSuccess) return (int)e;
      if ((e = cudaFuncSetAttribute(dense_gemm_kernel<256, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)dense_smem<256>())) != cudaSuccess) return (int)e;
      if ((e = cudaFuncSetAttribute(dense_gemm_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)dense_smem<128>())) != cudaSuccess) return (int)e;
      if ((e = cudaFuncSetAttribute(dense_gemm_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)dense_smem<128>())) != cudaSuccess) return (int)e;
      g_dense_sms[dev] = prop.multiProcessorCount;
      g_dense_attr[dev] = true;
    }
    sms = g_dense_sms[dev];
  }
  DenseParams p{};
  int rc = encode_bf16_rows(&p.a_map, x, T, K);
  if (rc) return rc;
  if ((rc = encode_bf16_rows(&p.w_map, w, N, K))) return rc;
  p.bias = bias;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.T = T;
  p.N = N;
  p.K = K;
  p.half = N / 2;
  p.ldo = swiglu ? N / 2 : N;
  p.status = status;
  // The wide tile (256 weight rows) halves the traffic of the token operand; it is used when it still gives every SM a
  // tile, otherwise the narrow one doubles the number of tiles.
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const int m_tiles = (T + DM - 1) / DM;
  if (swiglu) {
    const bool wide = (p.half % 128 == 0) && m_tiles * (p.half / 128) >= sms;
    return wide ? launch_dense<256, true>(p, sms, st) : launch_dense<128, true>(p, sms, st);
  }
  const bool wide = m_tiles * ((N + 255) / 256) >= sms;
  return wide ? launch_dense<256, false>(p, sms, st) : launch_dense<128, false>(p, sms, st);
}

extern "C" int b200moe_row_dot(const void* x, const void* w, void* out, int T, int K, void* stream) {
  if (T == 0) return 0;
  if (!x || !w || !out) return B200MOE_E_NULL;
  if (T < 0 || K < 8 || K % 8) return B200MOE_E_SHAPE;
  if (!aligned16(x) || !aligned16(w)) return B200MOE_E_ALIGN;
  row_dot_kernel<<<(unsigned)(((int64_t)T * 32 + 255) / 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(w), reinterpret_cast<__nv_bfloat16*>(out), T,
      K);
  return check_launch();
}
