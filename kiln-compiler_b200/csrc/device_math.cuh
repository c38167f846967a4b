// Scalar math of the fused kernels.  The closed forms are the ones the reference's generated
// kernels use (kiln/gpu/codegen.py:53-88): tanh through exp(-2|x|), erf by Abramowitz & Stegun
// 7.1.26, GELU in tanh or erf form.  Inside those forms exp and the division are the hardware
// approximations (ex2.approx, rcp.approx: relative error ~2^-22), which is also what the
// reference's `tl.exp` and `/` lower to; explicit DIV / EXP / SQRT ops of a graph stay IEEE.  The
// FP32 mode has to stay within 1e-5 of a float64 evaluation.
#pragma once

#include <cuda_runtime.h>
#include <math_constants.h>

#include "kb200_internal.h"

namespace kb200 {

__device__ __forceinline__ float d_tanh(float x) {
  float e = __expf(-2.0f * fabsf(x));
  float t = __fdividef(1.0f - e, 1.0f + e);
  return x < 0.0f ? -t : t;
}

__device__ __forceinline__ float d_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

__device__ __forceinline__ float d_erf(float x) {
  float a = fabsf(x);
  float t = __fdividef(1.0f, 1.0f + 0.3275911f * a);
  float p = t * (0.254829592f + t * (-0.284496736f + t * (1.421413741f + t * (-1.453152027f + t * 1.061405429f))));
  float y = 1.0f - p * __expf(-a * a);
  return x < 0.0f ? -y : y;
}

// tanh-GELU: 0.5 x (1 + tanh(u)), u = sqrt(2/pi) (x + 0.044715 x^3)  (kiln/gpu/codegen.py:70-75).
// Evaluated through the identity 0.5 (1 + tanh(u)) = 1 / (1 + exp(-2u)): the same function, in five
// FP32 instructions and two special-function ones (ex2, rcp) instead of seventeen and two -- the
// bias+GELU kernel was bound by instruction issue, not by memory.  exp(-2u) = 2^(x (k1 + k3 x^2)).
__device__ __forceinline__ float d_gelu_tanh(float x) {
  const float k1 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  const float k3 = k1 * 0.044715f;
  const float t = x * x;
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * fmaf(t, k3, k1)));   // +inf for very negative x, where the result is -0
  return __fdividef(x, 1.0f + e);
}

__device__ __forceinline__ float d_gelu_erf(float x) { return 0.5f * x * (1.0f + d_erf(x * 0.7071067811865476f)); }

// max/min that propagate NaN like NumPy's maximum/minimum (kiln/ir/ops.py:70-71).
__device__ __forceinline__ float d_max(float a, float b) { return (a != a || b != b) ? CUDART_NAN_F : fmaxf(a, b); }
__device__ __forceinline__ float d_min(float a, float b) { return (a != a || b != b) ? CUDART_NAN_F : fminf(a, b); }

__device__ __forceinline__ float apply_op(int opcode, float a, float b) {
  switch (opcode) {
    case KB200_OP_ADD: return a + b;
    case KB200_OP_SUB: return a - b;
    case KB200_OP_MUL: return a * b;
    case KB200_OP_DIV: return a / b;
    case KB200_OP_MAX: return d_max(a, b);
    case KB200_OP_MIN: return d_min(a, b);
    case KB200_OP_NEG: return -a;
    case KB200_OP_RELU: return d_max(a, 0.0f);
    case KB200_OP_EXP: return expf(a);
    case KB200_OP_TANH: return d_tanh(a);
    case KB200_OP_SIGMOID: return d_sigmoid(a);
    case KB200_OP_ERF: return d_erf(a);
    case KB200_OP_GELU_TANH: return d_gelu_tanh(a);
    case KB200_OP_GELU_ERF: return d_gelu_erf(a);
    case KB200_OP_RSQRT: return 1.0f / sqrtf(a);
    case KB200_OP_SQRT: return sqrtf(a);
    default: return a;  // COPY
  }
}

// One step of a chain on the running value v with side value s.
__device__ __forceinline__ float apply_chain(int op, float v, float s) {
  switch (op) {
    case CH_ADD: return v + s;
    case CH_SUB: return v - s;
    case CH_RSUB: return s - v;
    case CH_MUL: return v * s;
    case CH_DIV: return v / s;
    case CH_RDIV: return s / v;
    case CH_MAX: return d_max(v, s);
    case CH_MIN: return d_min(v, s);
    case CH_NEG: return -v;
    case CH_RELU: return d_max(v, 0.0f);
    case CH_EXP: return expf(v);
    case CH_TANH: return d_tanh(v);
    case CH_SIGMOID: return d_sigmoid(v);
    case CH_ERF: return d_erf(v);
    case CH_GELU_TANH: return d_gelu_tanh(v);
    case CH_GELU_ERF: return d_gelu_erf(v);
    case CH_RSQRT: return 1.0f / sqrtf(v);
    case CH_SQRT: return sqrtf(v);
    default: return v;
  }
}

// One chain step on N register-resident values: the switch is outside the element loop and every
// index is a compile-time constant, so v[] and side[] stay in registers and the N independent
// elements give the instruction-level parallelism.
template <int N>
__device__ __forceinline__ void chain_step(int op, float (&v)[N], const float (&side)[N]) {
#define KB200_EACH(expr)                  \
  _Pragma("unroll") for (int j = 0; j < N; ++j) { const float x = v[j]; const float s = side[j]; (void)s; v[j] = (expr); }
  switch (op) {
    case CH_ADD: KB200_EACH(x + s) break;
    case CH_SUB: KB200_EACH(x - s) break;
    case CH_RSUB: KB200_EACH(s - x) break;
    case CH_MUL: KB200_EACH(x * s) break;
    case CH_DIV: KB200_EACH(x / s) break;
    case CH_RDIV: KB200_EACH(s / x) break;
    case CH_MAX: KB200_EACH(d_max(x, s)) break;
    case CH_MIN: KB200_EACH(d_min(x, s)) break;
    case CH_NEG: KB200_EACH(-x) break;
    case CH_RELU: KB200_EACH(d_max(x, 0.0f)) break;
    case CH_EXP: KB200_EACH(expf(x)) break;
    case CH_TANH: KB200_EACH(d_tanh(x)) break;
    case CH_SIGMOID: KB200_EACH(d_sigmoid(x)) break;
    case CH_ERF: KB200_EACH(d_erf(x)) break;
    case CH_GELU_TANH: KB200_EACH(d_gelu_tanh(x)) break;
    case CH_GELU_ERF: KB200_EACH(d_gelu_erf(x)) break;
    case CH_RSQRT: KB200_EACH(1.0f / sqrtf(x)) break;
    case CH_SQRT: KB200_EACH(sqrtf(x)) break;
    default: break;
  }
#undef KB200_EACH
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace kb200
