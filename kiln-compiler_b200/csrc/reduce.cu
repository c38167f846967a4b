// Generic reduction: one reduce_sum / reduce_max over any set of dims that is not just the
// innermost one (column sums, full reductions).  Role of the reference's `reduction` generator
// (kiln/gpu/codegen.py:432-482).  Each CTA owns 32 neighbouring outputs; its 8 warps walk the
// reduced extent in parallel and combine through shared memory.  Neighbouring outputs sit on
// neighbouring lanes, so a reduction over leading dims (the kept dim is contiguous) is coalesced.
#include "device_math.cuh"
#include "kb200_internal.h"

namespace kb200 {

struct ReduceParams {
  int n_kept, n_red;
  int is_max;
  int64_t n_out, r_total;
  int64_t kept_shape[KB200_MAX_RANK], red_shape[KB200_MAX_RANK];
  int64_t x_kept_stride[KB200_MAX_RANK], x_red_stride[KB200_MAX_RANK], out_stride[KB200_MAX_RANK];
  const float* x;
  float* out;
};

__global__ void __launch_bounds__(256) reduce_generic_kernel(const __grid_constant__ ReduceParams p) {
  pdl_wait();                 // the producer of this kernel's inputs has completed
  pdl_launch_dependents();    // the next kernel may begin its start-up
  __shared__ float partial[8][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t groups = (p.n_out + 31) / 32;
  for (int64_t g = blockIdx.x; g < groups; g += gridDim.x) {
    const int64_t o = g * 32 + lane;
    float acc = p.is_max ? -CUDART_INF_F : 0.0f;
    int64_t out_off = 0;
    if (o < p.n_out) {
      int64_t x_off = 0, rest = o;
      for (int d = p.n_kept - 1; d >= 0; --d) {
        const int64_t i = rest % p.kept_shape[d];
        rest /= p.kept_shape[d];
        x_off += i * p.x_kept_stride[d];
        out_off += i * p.out_stride[d];
      }
      for (int64_t r = warp; r < p.r_total; r += 8) {
        int64_t off = x_off, rr = r;
        for (int d = p.n_red - 1; d >= 0; --d) {
          off += (rr % p.red_shape[d]) * p.x_red_stride[d];
          rr /= p.red_shape[d];
        }
        const float v = p.x[off];
        acc = p.is_max ? d_max(acc, v) : acc + v;
      }
    }
    partial[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && o < p.n_out) {
      float t = partial[0][lane];
#pragma unroll
      for (int w = 1; w < 8; ++w) t = p.is_max ? d_max(t, partial[w][lane]) : t + partial[w][lane];
      p.out[out_off] = t;
    }
    __syncthreads();
  }
}

int choose_reduce(Plan& plan, PlanKernel& k) {
  (void)plan;
  k.impl = IMPL_REDUCE_GENERIC;
  k.launches = 1;
  return KB200_OK;
}

int launch_reduce(const Plan& plan, const PlanKernel& k, cudaStream_t s) {
  const kb200_kernel_desc& d = k.desc;
  ReduceParams p{};
  const int x_slot = d.tape[0].a, out_slot = d.tape[2].b;
  p.n_kept = d.n_kept;
  p.n_red = d.iter_rank - d.n_kept;
  p.is_max = d.tape[1].opcode == KB200_OP_RMAX;
  p.n_out = 1;
  p.r_total = 1;
  for (int i = 0; i < p.n_kept; ++i) {
    p.kept_shape[i] = d.iter_shape[i];
    p.x_kept_stride[i] = k.ops[x_slot].stride[i];
    p.out_stride[i] = k.ops[out_slot].stride[i];
    p.n_out *= d.iter_shape[i];
  }
  for (int i = 0; i < p.n_red; ++i) {
    p.red_shape[i] = d.iter_shape[p.n_kept + i];
    p.x_red_stride[i] = k.ops[x_slot].stride[p.n_kept + i];
    p.r_total *= p.red_shape[i];
  }
  p.x = k.ops[x_slot].ptr;
  p.out = k.ops[out_slot].ptr;
  const int64_t groups = (p.n_out + 31) / 32;
  const int64_t cap = (int64_t)plan.sm_count * 8;
  launch_kernel(plan.pdl, reduce_generic_kernel, dim3((unsigned)(groups < cap ? groups : cap)), dim3(256), 0, s, p);
  KB200_CUDA(cudaGetLastError());
  return KB200_OK;
}

}  // namespace kb200
