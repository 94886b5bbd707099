// The decoder layer's glue around the MoE block: residual add fused with the RMSNorm that feeds the block
// (freetoken/python/freetoken/models/qwen3_5_moe/model.py:63-77 calls GemmaRMSNorm.forward_add_residual,
// freetoken/python/freetoken/layers/norm.py:72-76, whose kernel is freetoken/python/freetoken/kernel/triton/norm.py:78-111):
//   z = f32(x) + f32(residual);  residual = bf16(z);  x = bf16(z * rsqrt(mean(z*z) + eps) * (w [+ 1]))
// One warp per row, 16-byte loads and stores, the row held in registers between the two passes.
#include "common.cuh"

namespace b200moe {

template <bool ADD>
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(__nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ residual,
                                                           const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                                           float eps, int plus_one, int64_t rows, int H) {
  const int lane = threadIdx.x & 31;
  const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (row >= rows) return;
  constexpr int MAXV = 8;  // 16-byte pieces per lane held in registers: rows up to 2048 elements; longer rows re-read
  __nv_bfloat16* xr = x + row * H;
  __nv_bfloat16* rr = ADD ? residual + row * H : nullptr;
  float z[MAXV][8];
  float ss = 0.f;
  const int pieces = H >> 3;
  auto load_z = [&](int piece, float (&v)[8]) {
    const uint4 a = *reinterpret_cast<const uint4*>(xr + piece * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    uint32_t bw[4] = {0, 0, 0, 0};
    if (ADD) {
      const uint4 b = *reinterpret_cast<const uint4*>(rr + piece * 8);
      bw[0] = b.x; bw[1] = b.y; bw[2] = b.z; bw[3] = b.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = bf16_bits_to_float(aw[j] & 0xffffu) + (ADD ? bf16_bits_to_float(bw[j] & 0xffffu) : 0.f);
      v[2 * j + 1] = __uint_as_float(aw[j] & 0xffff0000u) + (ADD ? __uint_as_float(bw[j] & 0xffff0000u) : 0.f);
    }
  };
  for (int i = 0, piece = lane; piece < pieces; ++i, piece += 32) {
    float v[8];
    load_z(piece, v);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += v[j] * v[j];
    if (i < MAXV) {
#pragma unroll
      for (int j = 0; j < 8; ++j) z[i][j] = v[j];
    }
    if (ADD)  // the residual stream keeps the sum, rounded once
      *reinterpret_cast<uint4*>(rr + piece * 8) = make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                                              pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
  }
  ss = warp_sum(ss);
  const float inv = rsqrtf(ss / (float)H + eps);
  __nv_bfloat16* dst = (ADD ? xr : out + row * H);
  for (int i = 0, piece = lane; piece < pieces; ++i, piece += 32) {
    float v[8];
    if (i < MAXV) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = z[i][j];
    } else {
      // beyond the register window the row is read again (only the form without a residual gets here: its input
      // is untouched; the host refuses longer rows for the fused form, whose operands are overwritten in pass one)
      load_z(piece, v);
    }
    const uint4 wq = *reinterpret_cast<const uint4*>(w + piece * 8);
    const uint32_t ww[4] = {wq.x, wq.y, wq.z, wq.w};
    float y[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float w0 = bf16_bits_to_float(ww[j] & 0xffffu) + (plus_one ? 1.f : 0.f);
      const float w1 = __uint_as_float(ww[j] & 0xffff0000u) + (plus_one ? 1.f : 0.f);
      y[2 * j] = v[2 * j] * inv * w0;
      y[2 * j + 1] = v[2 * j + 1] * inv * w1;
    }
    *reinterpret_cast<uint4*>(dst + piece * 8) = make_uint4(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]),
                                                            pack_bf16x2(y[4], y[5]), pack_bf16x2(y[6], y[7]));
  }
}

}  // namespace b200moe

using namespace b200moe;

extern "C" int b200moe_fused_add_rmsnorm(void* x, void* residual, const void* weight, float eps, int plus_one, int64_t rows,
                                         int H, void* stream) {
  if (rows == 0) return 0;
  if (!x || !residual || !weight) return B200MOE_E_NULL;
  if (rows < 0 || H < 8 || H % 8 || H > 2048) return B200MOE_E_SHAPE;  // the sum of a row stays in registers
  if (!aligned16(x) || !aligned16(residual) || !aligned16(weight)) return B200MOE_E_ALIGN;
  const unsigned grid = (unsigned)((rows * 32 + 255) / 256);
  rmsnorm_rows_kernel<true><<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(residual),
      reinterpret_cast<const __nv_bfloat16*>(weight), nullptr, eps, plus_one, rows, H);
  return check_launch();
}

extern "C" int b200moe_rmsnorm(const void* x, const void* weight, void* out, float eps, int plus_one, int64_t rows, int H,
                               void* stream) {
  if (rows == 0) return 0;
  if (!x || !out || !weight) return B200MOE_E_NULL;
  if (rows < 0 || H < 8 || H % 8 || H > 16384) return B200MOE_E_SHAPE;
  if (!aligned16(x) || !aligned16(out) || !aligned16(weight)) return B200MOE_E_ALIGN;
  const unsigned grid = (unsigned)((rows * 32 + 255) / 256);
  rmsnorm_rows_kernel<false><<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      const_cast<__nv_bfloat16*>(reinterpret_cast<const __nv_bfloat16*>(x)), nullptr,
      reinterpret_cast<const __nv_bfloat16*>(weight), reinterpret_cast<__nv_bfloat16*>(out), eps, plus_one, rows, H);
  return check_launch();
}
