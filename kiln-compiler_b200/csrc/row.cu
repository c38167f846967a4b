// Row kernels: reductions over the innermost dim fused with the elementwise ops that share the
// rows (LayerNorm, softmax, row centring ...).  Role of the reference's `row` generator
// (kiln/gpu/codegen.py:312-430).
//
//   row_generic    any tape: one CTA per row, one pass over the row per level of reduction with
//                  the elementwise values recomputed from the inputs in every pass -- the scheme of
//                  the reference's chunked rows (codegen.py:371-428), so memory use is constant for
//                  any row length.
//   row_layernorm  two-pass mean / variance LayerNorm with affine, one warp per row, the row held
//   row_softmax    in registers (128-bit loads, shuffle reductions): one read and one write of
//                  the tensor, HBM-bound.
#include <cuda_bf16.h>

#include "device_math.cuh"
#include "kb200_internal.h"

namespace kb200 {

constexpr int kRowThreads = 256;
constexpr int kMaxRowRed = 8;

struct RowParams {
  int rank;                       // row dims + 1
  int n_operands;
  int max_level;
  int64_t n_rows;
  int64_t inner;
  int64_t shape[KB200_MAX_RANK];
  DevOperand ops[KB200_MAX_OPERANDS];
  DevTape tape;
};

__device__ __forceinline__ float block_reduce(float v, bool is_max, float* scratch) {
  v = is_max ? warp_max(v) : warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();                 // scratch may still be read from the previous reduction
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = lane < (kRowThreads / 32) ? scratch[lane] : (is_max ? -CUDART_INF_F : 0.0f);
  r = is_max ? warp_max(r) : warp_sum(r);
  return r;
}

__global__ void __launch_bounds__(kRowThreads) row_generic_kernel(const __grid_constant__ RowParams p) {
  pdl_wait();                 // the producer of this kernel's inputs has completed
  pdl_launch_dependents();    // the next kernel may begin its start-up
  __shared__ float s_red[KB200_MAX_TAPE];
  __shared__ float s_scratch[kRowThreads / 32];
  float r[KB200_MAX_TAPE];
  int64_t rowoff[KB200_MAX_OPERANDS];
  const int inner_d = p.rank - 1;
  for (int64_t row = blockIdx.x; row < p.n_rows; row += gridDim.x) {
    for (int o = 0; o < p.n_operands; ++o) rowoff[o] = 0;
    int64_t rest = row;
    for (int d = inner_d - 1; d >= 0; --d) {
      int64_t i = rest % p.shape[d];
      rest /= p.shape[d];
      for (int o = 0; o < p.n_operands; ++o) rowoff[o] += i * p.ops[o].stride[d];
    }
    // pass `limit` evaluates every value below that level; the last pass also stores
    for (int limit = 1; limit <= p.max_level + 1; ++limit) {
      const bool final_pass = limit == p.max_level + 1;
      int red_idx[kMaxRowRed];
      float acc[kMaxRowRed];
      int n_red = 0;
      if (!final_pass) {
        for (int t = 0; t < p.tape.n; ++t) {
          const int oc = p.tape.ops[t].opcode;
          if ((oc == KB200_OP_RSUM || oc == KB200_OP_RMAX) && p.tape.ops[t].level == limit && n_red < kMaxRowRed) {
            red_idx[n_red] = t;
            acc[n_red] = oc == KB200_OP_RSUM ? 0.0f : -CUDART_INF_F;
            ++n_red;
          }
        }
      }
      for (int64_t col = threadIdx.x; col < p.inner; col += kRowThreads) {
        for (int t = 0; t < p.tape.n; ++t) {
          const kb200_tape_op op = p.tape.ops[t];
          if (op.opcode == KB200_OP_STORE) {
            if (final_pass) {
              const int64_t st = p.ops[op.b].stride[inner_d];
              if (st != 0 || col == 0) p.ops[op.b].ptr[rowoff[op.b] + col * st] = r[op.a];
            }
            continue;
          }
          if (op.level >= limit) continue;
          switch (op.opcode) {
            case KB200_OP_LOAD: r[t] = p.ops[op.a].ptr[rowoff[op.a] + col * p.ops[op.a].stride[inner_d]]; break;
            case KB200_OP_IMM: r[t] = op.imm; break;
            case KB200_OP_RSUM:
            case KB200_OP_RMAX: r[t] = s_red[t]; break;
            default: r[t] = apply_op(op.opcode, r[op.a], r[op.b]); break;
          }
        }
        for (int j = 0; j < n_red; ++j) {
          const kb200_tape_op op = p.tape.ops[red_idx[j]];
          const float v = r[op.a];
          acc[j] = op.opcode == KB200_OP_RSUM ? acc[j] + v : d_max(acc[j], v);
        }
      }
      for (int j = 0; j < n_red; ++j) {
        const bool is_max = p.tape.ops[red_idx[j]].opcode == KB200_OP_RMAX;
        const float total = block_reduce(acc[j], is_max, s_scratch);
        if (threadIdx.x == 0) s_red[red_idx[j]] = total;
      }
      __syncthreads();
    }
  }
}

// ---- register-resident rows: LayerNorm and softmax ----
struct RowFastParams {
  const float* x;
  float* out;
  const float* gamma;
  const float* beta;
  int64_t n_rows;
  int64_t x_row_stride, out_row_stride;
  int inner;
  float inv_n, eps;
  __nv_bfloat16* out16;    // optional bf16 copy of the output (same row stride as `out`), or null
  int store32;             // 0: only that copy is stored (every reader of the output takes it)
  // Two row dims (a [batch * heads, tokens, inner] softmax whose mask varies with the token only):
  // row = i0 * rows_inner + i1, and every tensor has a stride for each.  rows_inner == 0: one row dim.
  int64_t rows_inner;
  int64_t x_stride1, out_stride1;
  // A short elementwise chain applied to the loaded row before the reductions (scale and additive
  // mask in front of a softmax, a residual add in front of a LayerNorm), and where to store its value.
  int n_pre;
  struct Pre {
    int op;                // ChainOp
    int kind;              // 0 unary, 1 immediate, 2 tensor
    float imm;
    const float* ptr;
    int64_t stride0, stride1;
    int inner_stride;      // 1, or 0 for one value per row
  } pre[kMaxRowPre];
  float* pre_out;          // receives the chain's value (same shape as x), or null
  int64_t pre_out_stride0, pre_out_stride1;
};

enum { ROW_LAYERNORM = 0, ROW_SOFTMAX = 1 };

// One warp per row; lane l owns float4 number l + 32 * i, i < VPL.
template <int MODE, int VPL>
__global__ void __launch_bounds__(256) row_warp_kernel(const __grid_constant__ RowFastParams p) {
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const int64_t row = (int64_t)blockIdx.x * warps + (threadIdx.x >> 5);
  const int nvec = p.inner >> 2;
  // The affine parameters of a LayerNorm are constants of the plan, not outputs of the previous
  // kernel: they are fetched before this kernel waits for its producer, so their latency is off the
  // path (fetched after the two reductions they added a dependent memory round trip to every row).
  float4 g[MODE == ROW_LAYERNORM ? VPL : 1], b[MODE == ROW_LAYERNORM ? VPL : 1];
  if (MODE == ROW_LAYERNORM) {
    const float4* g4 = reinterpret_cast<const float4*>(p.gamma);
    const float4* b4 = reinterpret_cast<const float4*>(p.beta);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      const int j = lane + 32 * i;
      if (j < nvec) { g[i] = __ldg(g4 + j); b[i] = __ldg(b4 + j); }
    }
  }
  pdl_wait();                 // the producer of this kernel's inputs has completed
  pdl_launch_dependents();    // the next kernel may begin its start-up
  if (row >= p.n_rows) return;
  int64_t i0 = row, i1 = 0;
  if (p.rows_inner > 0) { i0 = row / p.rows_inner; i1 = row - i0 * p.rows_inner; }
  const float4* x4 = reinterpret_cast<const float4*>(p.x + i0 * p.x_row_stride + i1 * p.x_stride1);
  float4* o4 = reinterpret_cast<float4*>(p.out + i0 * p.out_row_stride + i1 * p.out_stride1);
  const int64_t out16_off = i0 * p.out_row_stride + i1 * p.out_stride1;
  float4 v[VPL];
  bool live[VPL];
#pragma unroll
  for (int i = 0; i < VPL; ++i) {
    const int j = lane + 32 * i;
    live[i] = j < nvec;
    if (live[i]) v[i] = x4[j];
  }
  for (int s = 0; s < p.n_pre; ++s) {
    const RowFastParams::Pre st = p.pre[s];
    const float* side = st.kind == 2 ? st.ptr + i0 * st.stride0 + i1 * st.stride1 : nullptr;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (!live[i]) continue;
      float4 t = make_float4(st.imm, st.imm, st.imm, st.imm);
      if (st.kind == 2) {
        if (st.inner_stride == 1) t = *reinterpret_cast<const float4*>(side + 4 * (lane + 32 * i));
        else { const float one = __ldg(side); t = make_float4(one, one, one, one); }
      }
      v[i].x = apply_chain(st.op, v[i].x, t.x);
      v[i].y = apply_chain(st.op, v[i].y, t.y);
      v[i].z = apply_chain(st.op, v[i].z, t.z);
      v[i].w = apply_chain(st.op, v[i].w, t.w);
    }
  }
  if (p.pre_out != nullptr) {
    float4* z4 = reinterpret_cast<float4*>(p.pre_out + i0 * p.pre_out_stride0 + i1 * p.pre_out_stride1);
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (live[i]) z4[lane + 32 * i] = v[i];
  }
  if (MODE == ROW_LAYERNORM) {
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (live[i]) s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
    const float mean = warp_sum(s) * p.inv_n;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (live[i]) {
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        q += (v[i].x * v[i].x + v[i].y * v[i].y) + (v[i].z * v[i].z + v[i].w * v[i].w);
      }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(q) * p.inv_n + p.eps);
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (live[i]) {
        const int j = lane + 32 * i;
        float4 y;
        y.x = v[i].x * rstd * g[i].x + b[i].x;
        y.y = v[i].y * rstd * g[i].y + b[i].y;
        y.z = v[i].z * rstd * g[i].z + b[i].z;
        y.w = v[i].w * rstd * g[i].w + b[i].w;
        if (p.store32) o4[j] = y;
        if (p.out16 != nullptr) {
          __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y), hi = __floats2bfloat162_rn(y.z, y.w);
          uint2 packed;
          packed.x = *reinterpret_cast<uint32_t*>(&lo);
          packed.y = *reinterpret_cast<uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(p.out16 + out16_off + 4 * j) = packed;
        }
      }
    }
  } else {
    float m = -CUDART_INF_F;
#pragma unroll
    for (int i = 0; i < VPL; ++i)
      if (live[i]) m = fmaxf(m, fmaxf(fmaxf(v[i].x, v[i].y), fmaxf(v[i].z, v[i].w)));
    m = warp_max(m);
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (live[i]) {
        // exp through ex2.approx (relative error 2^-22, what the reference's tl.exp lowers to as well)
        v[i].x = __expf(v[i].x - m); v[i].y = __expf(v[i].y - m); v[i].z = __expf(v[i].z - m); v[i].w = __expf(v[i].w - m);
        s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
      }
    }
    s = warp_sum(s);
    const float inv = 1.0f / s;     // one IEEE division per row; the elements are scaled by it (within an ulp of dividing)
#pragma unroll
    for (int i = 0; i < VPL; ++i) {
      if (live[i]) {
        float4 y;
        y.x = v[i].x * inv; y.y = v[i].y * inv; y.z = v[i].z * inv; y.w = v[i].w * inv;
        o4[lane + 32 * i] = y;
      }
    }
  }
}

template <int MODE>
static void launch_row_warp(const RowFastParams& p, int sm_count, bool pdl, cudaStream_t s) {
  const int vpl = (p.inner / 4 + 31) / 32;
  int warps = p.n_rows >= (int64_t)sm_count * 16 ? 8 : (p.n_rows >= (int64_t)sm_count * 4 ? 4 : 1);
  const unsigned grid = (unsigned)((p.n_rows + warps - 1) / warps);
  const unsigned block = warps * 32;
#define KB200_ROW_CASE(V) launch_kernel(pdl, row_warp_kernel<MODE, V>, dim3(grid), dim3(block), 0, s, p)
  if (vpl <= 1) KB200_ROW_CASE(1);
  else if (vpl <= 2) KB200_ROW_CASE(2);
  else if (vpl <= 4) KB200_ROW_CASE(4);
  else if (vpl <= 6) KB200_ROW_CASE(6);
  else if (vpl <= 8) KB200_ROW_CASE(8);
  else if (vpl <= 12) KB200_ROW_CASE(12);
  else KB200_ROW_CASE(16);
#undef KB200_ROW_CASE
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int choose_row(Plan& plan, PlanKernel& k) {
  (void)plan;
  const kb200_kernel_desc& d = k.desc;
  k.impl = IMPL_ROW_GENERIC;
  k.launches = 1;
  // the generic kernel keeps at most kMaxRowRed running reductions per pass (one pass per level)
  int per_level[KB200_MAX_TAPE + 1] = {0};
  for (int t = 0; t < d.n_tape; ++t) {
    const int oc = d.tape[t].opcode;
    if (oc != KB200_OP_RSUM && oc != KB200_OP_RMAX) continue;
    const int level = d.tape[t].level;
    if (level < 0 || level > KB200_MAX_TAPE)
      return fail(KB200_ERR_ARGUMENT, "row kernel %s: reduction level %d out of range", d.name, level);
    if (++per_level[level] > kMaxRowRed)
      return fail(KB200_ERR_UNSUPPORTED, "row kernel %s: more than %d reductions at one level of the chain", d.name, kMaxRowRed);
  }
  const int64_t inner = d.iter_shape[d.iter_rank - 1];
  // register-resident rows: one or two row dims, rows of 4..2048 floats in 128-bit units
  const int last = d.iter_rank - 1;
  const bool shape_ok = (d.iter_rank == 2 || d.iter_rank == 3) && inner % 4 == 0 && inner <= 2048 && inner >= 4;
  if (!shape_ok) return KB200_OK;
  auto row_tensor_ok = [&](int slot) {
    const DevOperand& o = k.ops[slot];
    if (o.stride[last] != 1 || !aligned16(o.ptr)) return false;
    for (int dd = 0; dd < last; ++dd)
      if (o.stride[dd] % 4) return false;
    return true;
  };
  auto vector_ok = [&](int slot) {
    const DevOperand& o = k.ops[slot];
    if (o.stride[last] != 1 || !aligned16(o.ptr)) return false;
    for (int dd = 0; dd < last; ++dd)
      if (o.stride[dd] != 0) return false;
    return true;
  };
  // operands of the chain in front of the reductions: a tensor like x, or one value per row
  auto pre_ok = [&]() {
    for (int st = 0; st < k.row_pre.n; ++st) {
      const int slot = k.row_pre.steps[st].slot;
      if (slot < 0) continue;
      const DevOperand& o = k.ops[slot];
      if (o.stride[last] == 0) continue;
      if (!row_tensor_ok(slot)) return false;
    }
    return k.pre_out_slot < 0 || row_tensor_ok(k.pre_out_slot);
  };
  k.row_pre.n = 0;
  k.pre_out_slot = -1;
  if (match_layernorm(d, &k)) {
    if (row_tensor_ok(k.x_slot) && row_tensor_ok(k.out_slot) && vector_ok(k.g_slot) && vector_ok(k.b_slot) && pre_ok())
      k.impl = IMPL_ROW_LAYERNORM;
  } else if (match_softmax(d, &k)) {
    if (row_tensor_ok(k.x_slot) && row_tensor_ok(k.out_slot) && pre_ok()) k.impl = IMPL_ROW_SOFTMAX;
  }
  return KB200_OK;
}

int launch_row(const Plan& plan, const PlanKernel& k, cudaStream_t s) {
  const kb200_kernel_desc& d = k.desc;
  const int64_t inner = d.iter_shape[d.iter_rank - 1];
  int64_t n_rows = 1;
  for (int i = 0; i < d.iter_rank - 1; ++i) n_rows *= d.iter_shape[i];
  if (k.impl == IMPL_ROW_LAYERNORM || k.impl == IMPL_ROW_SOFTMAX) {
    RowFastParams p{};
    p.store32 = 1;
    p.x = k.ops[k.x_slot].ptr;
    p.out = k.ops[k.out_slot].ptr;
    p.n_rows = n_rows;
    p.x_row_stride = k.ops[k.x_slot].stride[0];
    p.out_row_stride = k.ops[k.out_slot].stride[0];
    p.inner = (int)inner;
    const bool two = d.iter_rank == 3;
    p.rows_inner = two ? d.iter_shape[1] : 0;
    p.x_stride1 = two ? k.ops[k.x_slot].stride[1] : 0;
    p.out_stride1 = two ? k.ops[k.out_slot].stride[1] : 0;
    p.n_pre = k.row_pre.n;
    for (int st = 0; st < k.row_pre.n; ++st) {
      const ChainStep& cs = k.row_pre.steps[st];
      RowFastParams::Pre& pr = p.pre[st];
      pr.op = cs.op;
      pr.imm = cs.imm;
      pr.kind = cs.slot == -2 ? 0 : (cs.slot == -1 ? 1 : 2);
      if (cs.slot >= 0) {
        const DevOperand& o = k.ops[cs.slot];
        pr.ptr = o.ptr;
        pr.stride0 = o.stride[0];
        pr.stride1 = two ? o.stride[1] : 0;
        pr.inner_stride = (int)o.stride[d.iter_rank - 1];
      }
    }
    p.pre_out = k.pre_out_slot >= 0 ? k.ops[k.pre_out_slot].ptr : nullptr;
    p.pre_out_stride0 = k.pre_out_slot >= 0 ? k.ops[k.pre_out_slot].stride[0] : 0;
    p.pre_out_stride1 = k.pre_out_slot >= 0 && two ? k.ops[k.pre_out_slot].stride[1] : 0;
    if (k.impl == IMPL_ROW_LAYERNORM) {
      p.gamma = k.ops[k.g_slot].ptr;
      p.beta = k.ops[k.b_slot].ptr;
      p.inv_n = k.ln_inv_n;
      p.eps = k.ln_eps;
      p.out16 = static_cast<__nv_bfloat16*>(k.shadow_out);
      p.store32 = (k.mirror_only && p.out16 != nullptr) ? 0 : 1;
      launch_row_warp<ROW_LAYERNORM>(p, plan.sm_count, plan.pdl, s);
    } else {
      launch_row_warp<ROW_SOFTMAX>(p, plan.sm_count, plan.pdl, s);
    }
  } else {
    RowParams p{};
    p.rank = d.iter_rank;
    p.n_operands = d.n_operands;
    p.n_rows = n_rows;
    p.inner = inner;
    p.max_level = 0;
    for (int t = 0; t < d.n_tape; ++t)
      if (d.tape[t].level > p.max_level) p.max_level = d.tape[t].level;
    for (int i = 0; i < d.iter_rank; ++i) p.shape[i] = d.iter_shape[i];
    for (int o = 0; o < d.n_operands; ++o) p.ops[o] = k.ops[o];
    p.tape = k.tape;
    int64_t cap = (int64_t)plan.sm_count * 8;
    launch_kernel(plan.pdl, row_generic_kernel, dim3((unsigned)(n_rows < cap ? n_rows : cap)), dim3(kRowThreads), 0, s, p);
  }
  KB200_CUDA(cudaGetLastError());
  return KB200_OK;
}

}  // namespace kb200
