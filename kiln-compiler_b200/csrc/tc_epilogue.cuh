// Epilogue arithmetic shared by the tensor-core matmul kernels: the closed forms of the fused scalar
// ops on 32 register-resident values, and the staging of a 32 x 32 block for a bulk tensor store.
#pragma once

#include <cuda_bf16.h>

#include "device_math.cuh"
#include "kb200_internal.h"

namespace kb200 {
namespace tc {

// Reduced-precision modes only: exp through ex2.approx and division through rcp.approx (relative
// error ~1e-6, far inside the 2e-3 / 2e-2 budgets of TF32 / BF16 operands).  The closed forms stay
// the reference's (kiln/gpu/codegen.py:53-88).
__device__ __forceinline__ float f_tanh(float x) {
  const float e = __expf(-2.0f * fabsf(x));
  const float t = __fdividef(1.0f - e, 1.0f + e);
  return x < 0.0f ? -t : t;
}
// BF16 mode only: one MUFU instruction (relative error 2^-11; the block's output moves by 1e-3 of its
// scale, against a budget of 2e-2) instead of ex2 + rcp.  The GELU epilogue of a 128 x 256 tile is bound
// by the MUFU and issue rates of its eight warps: this takes 2 us off the block's 768 -> 3072 layer.
__device__ __forceinline__ float f_tanh_approx(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 0.5 x (1 + tanh(k (x + c x^3))) in six instructions: the polynomial by one multiply-add on x^2, the
// final product as h + h t with h = x / 2.
__device__ __forceinline__ float f_gelu_tanh_approx(float x) {
  const float x2 = x * x;
  const float u = x * fmaf(x2, 0.7978845608028654f * 0.044715f, 0.7978845608028654f);
  const float h = 0.5f * x;
  return fmaf(h, f_tanh_approx(u), h);
}

__device__ __forceinline__ float f_erf(float x) {
  const float a = fabsf(x);
  const float t = __fdividef(1.0f, 1.0f + 0.3275911f * a);
  const float p = t * (0.254829592f + t * (-0.284496736f + t * (1.421413741f + t * (-1.453152027f + t * 1.061405429f))));
  const float y = 1.0f - p * __expf(-a * a);
  return x < 0.0f ? -y : y;
}

// One chain step on a single value (the split-K reduction works on float4 items): the BF16-mode
// approximations here, everything else as the CUDA-core kernels evaluate it.
__device__ __forceinline__ float chain_apply_scalar(int op, float v, float s) {
  if (op == CH_TANH_APPROX) return f_tanh_approx(v);
  if (op == CH_GELU_TANH_APPROX) return f_gelu_tanh_approx(v);
  return apply_chain(op, v, s);
}

// The two GELU forms on W register-resident values, written stage by stage over groups of eight
// elements: eight independent multiply-adds, then eight special-function instructions, ...  Written
// element by element (the whole formula for one value, then the next) the compiled code kept that order:
// every instruction waited out the latency of the one before it, special-function unit included, ~57
// cycles per value and lane in the epilogue of the 768 -> 3072 layer.
template <int W>
__device__ __forceinline__ void gelu_tanh_approx_n(float (&v)[W]) {
#pragma unroll
  for (int g = 0; g < W; g += 8) {
    float u[8], h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = v[g + j] * v[g + j];
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = fmaf(u[j], 0.7978845608028654f * 0.044715f, 0.7978845608028654f);
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = v[g + j] * u[j];
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = f_tanh_approx(u[j]);
#pragma unroll
    for (int j = 0; j < 8; ++j) h[j] = 0.5f * v[g + j];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[g + j] = fmaf(h[j], u[j], h[j]);
  }
}
// x / (1 + 2^(x (k1 + k3 x^2))), the closed form of d_gelu_tanh
template <int W>
__device__ __forceinline__ void gelu_tanh_n(float (&v)[W]) {
  const float k1 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  const float k3 = k1 * 0.044715f;
#pragma unroll
  for (int g = 0; g < W; g += 8) {
    float u[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = v[g + j] * v[g + j];
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = fmaf(u[j], k3, k1);
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = v[g + j] * u[j];
#pragma unroll
    for (int j = 0; j < 8; ++j) asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(u[j]) : "f"(u[j]));
#pragma unroll
    for (int j = 0; j < 8; ++j) u[j] = 1.0f + u[j];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[g + j] = __fdividef(v[g + j], u[j]);
  }
}

// One chain step on W register-resident values.  The switch is outside the element loop and
// every index is a compile-time constant, so v[] and side[] never leave the register file and the
// W independent elements give the few epilogue warps the instruction-level parallelism they need.
template <int W>
__device__ __forceinline__ void chain_step_n(int op, float (&v)[W], const float (&side)[W]) {
#define KB200_EACH(expr)                  \
  _Pragma("unroll") for (int j = 0; j < W; ++j) { const float x = v[j]; const float s = side[j]; (void)s; v[j] = (expr); }
  switch (op) {
    case CH_ADD: KB200_EACH(x + s) break;
    case CH_SUB: KB200_EACH(x - s) break;
    case CH_RSUB: KB200_EACH(s - x) break;
    case CH_MUL: KB200_EACH(x * s) break;
    case CH_DIV: KB200_EACH(__fdividef(x, s)) break;
    case CH_RDIV: KB200_EACH(__fdividef(s, x)) break;
    case CH_MAX: KB200_EACH(d_max(x, s)) break;
    case CH_MIN: KB200_EACH(d_min(x, s)) break;
    case CH_NEG: KB200_EACH(-x) break;
    case CH_RELU: KB200_EACH(d_max(x, 0.0f)) break;
    case CH_EXP: KB200_EACH(__expf(x)) break;
    case CH_TANH: KB200_EACH(f_tanh(x)) break;
    case CH_SIGMOID: KB200_EACH(__fdividef(1.0f, 1.0f + __expf(-x))) break;
    case CH_ERF: KB200_EACH(f_erf(x)) break;
    case CH_GELU_TANH: gelu_tanh_n<W>(v); break;
    case CH_GELU_ERF: KB200_EACH(0.5f * x * (1.0f + f_erf(x * 0.7071067811865476f))) break;
    case CH_TANH_APPROX: KB200_EACH(f_tanh_approx(x)) break;
    case CH_GELU_TANH_APPROX: gelu_tanh_approx_n<W>(v); break;
    case CH_RSQRT: KB200_EACH(rsqrtf(x)) break;
    case CH_SQRT: KB200_EACH(sqrtf(x)) break;
    default: break;
  }
#undef KB200_EACH
}
__device__ __forceinline__ void chain_step32(int op, float (&v)[32], const float (&side)[32]) { chain_step_n<32>(op, v, side); }

// Staging of a 32 x 32 block for the bulk stores with a lane per ROW (v[j] = column j), in the swizzled
// layouts of the store maps: float rows of 128 bytes with the 16-byte unit index XORed by (row & 7),
// bf16 rows of 64 bytes with the unit index XORed by ((row >> 1) & 3).  128-bit stores, no bank conflicts.
__device__ __forceinline__ void stage_rows(uint8_t* sf, uint8_t* sh, const float (&v)[32], int lane, bool with16, bool with32 = true) {
  if (with32) {
#pragma unroll
    for (int q = 0; q < 8; ++q)
      *reinterpret_cast<float4*>(sf + lane * 128 + ((q ^ (lane & 7)) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  }
  if (with16) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      __nv_bfloat162 w0 = __floats2bfloat162_rn(v[8 * q], v[8 * q + 1]), w1 = __floats2bfloat162_rn(v[8 * q + 2], v[8 * q + 3]);
      __nv_bfloat162 w2 = __floats2bfloat162_rn(v[8 * q + 4], v[8 * q + 5]), w3 = __floats2bfloat162_rn(v[8 * q + 6], v[8 * q + 7]);
      uint4 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&w0);
      packed.y = *reinterpret_cast<uint32_t*>(&w1);
      packed.z = *reinterpret_cast<uint32_t*>(&w2);
      packed.w = *reinterpret_cast<uint32_t*>(&w3);
      *reinterpret_cast<uint4*>(sh + lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4)) = packed;
    }
  }
}

// Two 32 x 32 blocks side by side (columns 0-31 in v, 32-63 in w) as one 32 x 64 bf16 box: rows of 128
// bytes, the 16-byte unit index XORed by (row & 7).
__device__ __forceinline__ void stage_rows_bf16x64(uint8_t* sh, const float (&v)[32], const float (&w)[32], int lane) {
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    const float* x = q < 4 ? &v[8 * q] : &w[8 * (q - 4)];
    __nv_bfloat162 w0 = __floats2bfloat162_rn(x[0], x[1]), w1 = __floats2bfloat162_rn(x[2], x[3]);
    __nv_bfloat162 w2 = __floats2bfloat162_rn(x[4], x[5]), w3 = __floats2bfloat162_rn(x[6], x[7]);
    uint4 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&w0);
    packed.y = *reinterpret_cast<uint32_t*>(&w1);
    packed.z = *reinterpret_cast<uint32_t*>(&w2);
    packed.w = *reinterpret_cast<uint32_t*>(&w3);
    *reinterpret_cast<uint4*>(sh + lane * 128 + ((q ^ (lane & 7)) << 4)) = packed;
  }
}

}  // namespace tc
}  // namespace kb200
