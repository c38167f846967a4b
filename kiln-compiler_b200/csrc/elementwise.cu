// Elementwise kernels: fused chains of scalar ops over strided / broadcast operands, and copies.
// Role of the reference's `elementwise` generator (kiln/gpu/codegen.py:284-310).
//
//   ew_generic      any tape, any strides: one element per thread, values in a per-thread file.
//   ew_chain_vec4   the tape is a chain and every operand is contiguous (or constant) along the
//                   innermost dim: 128-bit loads/stores, the running value stays in registers.
//                   HBM-bound: reads each input once, writes the output once.
//   ew_transpose    a chain whose first input is contiguous along a different dim than the output
//                   (head-split K^T copy, unfrozen weight transposes): 32x32 tiles through shared
//                   memory so both the read and the write are coalesced.
#include "device_math.cuh"
#include "kb200_internal.h"

namespace kb200 {

struct EwParams {
  int rank;
  int n_operands;
  int64_t numel;
  int64_t shape[KB200_MAX_RANK];
  DevOperand ops[KB200_MAX_OPERANDS];
  DevTape tape;
};

__global__ void __launch_bounds__(256) ew_generic_kernel(const __grid_constant__ EwParams p) {
  pdl_wait();                 // the producer of this kernel's inputs has completed
  pdl_launch_dependents();    // the next kernel may begin its start-up
  float r[KB200_MAX_TAPE];
  int64_t off[KB200_MAX_OPERANDS];
  const int64_t step = (int64_t)gridDim.x * blockDim.x;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < p.numel; idx += step) {
    for (int o = 0; o < p.n_operands; ++o) off[o] = 0;
    int64_t rest = idx;
    for (int d = p.rank - 1; d >= 0; --d) {
      int64_t i = rest % p.shape[d];
      rest /= p.shape[d];
      for (int o = 0; o < p.n_operands; ++o) off[o] += i * p.ops[o].stride[d];
    }
    for (int t = 0; t < p.tape.n; ++t) {
      const kb200_tape_op op = p.tape.ops[t];
      switch (op.opcode) {
        case KB200_OP_LOAD: r[t] = p.ops[op.a].ptr[off[op.a]]; break;
        case KB200_OP_IMM: r[t] = op.imm; break;
        case KB200_OP_STORE: p.ops[op.b].ptr[off[op.b]] = r[op.a]; break;
        default: r[t] = apply_op(op.opcode, r[op.a], r[op.b]); break;
      }
    }
  }
}

// ---- vectorised chain ----
constexpr int kVecRank = 4;

struct EwChainParams {
  uint32_t nvec;
  uint32_t shape[kVecRank];      // last entry = inner / 4
  float* ptr[KB200_MAX_OPERANDS];
  // element strides as 32-bit numbers (the host takes this kernel only when every offset fits),
  // the innermost one already multiplied by 4: 4 (a float4 per index) or 0 (one scalar per row)
  int32_t stride[KB200_MAX_OPERANDS][kVecRank];
  Chain chain;
};

template <int RANK>
__device__ __forceinline__ uint32_t ew_offset(const EwChainParams& p, int slot, const uint32_t* idx) {
  uint32_t off = 0;
#pragma unroll
  for (int d = 0; d < RANK; ++d) off += idx[d] * (uint32_t)p.stride[slot][d];
  return off;
}

template <int RANK>
__device__ __forceinline__ float4 ew_load4(const EwChainParams& p, int slot, const uint32_t* idx) {
  const float* ptr = p.ptr[slot] + ew_offset<RANK>(p, slot, idx);
  if (p.stride[slot][RANK - 1] == 0) {
    float s = __ldg(ptr);
    return make_float4(s, s, s, s);
  }
  return *reinterpret_cast<const float4*>(ptr);
}

// U float4 per thread, a block's vectors contiguous per u (coalesced).  The rank is a template
// parameter and all index arithmetic is 32-bit: at 8 bytes moved per element the kernel must stay
// far below the instruction budget of the memory system (a generic 64-bit version of the same loop
// spent 75 instructions per element and ran at a third of the copy bandwidth).
template <int RANK, int U>
__global__ void __launch_bounds__(256) ew_chain_vec4_kernel(const __grid_constant__ EwChainParams p) {
  pdl_wait();                 // the producer of this kernel's inputs has completed
  pdl_launch_dependents();    // the next kernel may begin its start-up
  const uint32_t nvec = p.nvec;
  const uint32_t step = gridDim.x * blockDim.x * U;
  for (uint32_t base = blockIdx.x * blockDim.x * U + threadIdx.x; base < nvec; base += step) {
    float v[4 * U];
    uint32_t idx[U][RANK];
    bool live[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = base + (uint32_t)u * blockDim.x;
      live[u] = i < nvec;
      uint32_t rest = live[u] ? i : 0;
#pragma unroll
      for (int d = RANK - 1; d > 0; --d) {
        const uint32_t q = rest / p.shape[d];
        idx[u][d] = rest - q * p.shape[d];
        rest = q;
      }
      idx[u][0] = rest;
      const float4 x = live[u] ? ew_load4<RANK>(p, p.chain.first_slot, idx[u]) : make_float4(0.f, 0.f, 0.f, 0.f);
      v[4 * u] = x.x; v[4 * u + 1] = x.y; v[4 * u + 2] = x.z; v[4 * u + 3] = x.w;
    }
    for (int s = 0; s < p.chain.n; ++s) {
      const ChainStep st = p.chain.steps[s];
      float side[4 * U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float4 x = make_float4(st.imm, st.imm, st.imm, st.imm);
        if (st.slot >= 0 && live[u]) x = ew_load4<RANK>(p, st.slot, idx[u]);
        side[4 * u] = x.x; side[4 * u + 1] = x.y; side[4 * u + 2] = x.z; side[4 * u + 3] = x.w;
      }
      chain_step<4 * U>(st.op, v, side);
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (live[u])
        *reinterpret_cast<float4*>(p.ptr[p.chain.out_slot] + ew_offset<RANK>(p, p.chain.out_slot, idx[u])) =
            make_float4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
  }
}

// ---- tiled transpose + chain ----
struct EwTransposeParams {
  int rank;                      // 2..kVecRank
  int tdim;                      // the dim along which the first input is contiguous (!= rank - 1)
  int64_t shape[kVecRank];
  int64_t outer;                 // product of the dims other than tdim and the last
  DevOperand ops[KB200_MAX_OPERANDS];
  Chain chain;
};

__global__ void __launch_bounds__(256) ew_transpose_kernel(const __grid_constant__ EwTransposeParams p) {
  pdl_wait();                 // the producer of this kernel's inputs has completed
  pdl_launch_dependents();    // the next kernel may begin its start-up
  __shared__ float tile[32][33];
  const int last = p.rank - 1;
  const int64_t n_t = p.shape[p.tdim], n_l = p.shape[last];
  const int64_t tiles_l = (n_l + 31) / 32, tiles_t = (n_t + 31) / 32;
  const int64_t total = tiles_l * tiles_t * p.outer;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
  for (int64_t tile_id = blockIdx.x; tile_id < total; tile_id += gridDim.x) {
    int64_t rest = tile_id;
    const int64_t tl = rest % tiles_l; rest /= tiles_l;
    const int64_t tt = rest % tiles_t; rest /= tiles_t;
    int64_t idx[kVecRank] = {0, 0, 0, 0};
#pragma unroll
    for (int d = kVecRank - 1; d >= 0; --d) {
      if (d < p.rank && d != p.tdim && d != last) {
        idx[d] = rest % p.shape[d];
        rest /= p.shape[d];
      }
    }
    int64_t in_base = 0;
#pragma unroll
    for (int d = 0; d < kVecRank; ++d)
      if (d < p.rank) in_base += idx[d] * p.ops[p.chain.first_slot].stride[d];
    const int64_t s_t = p.ops[p.chain.first_slot].stride[p.tdim], s_l = p.ops[p.chain.first_slot].stride[last];
    // read: threads run along tdim (contiguous in the input)
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      int64_t it = tt * 32 + tx, il = tl * 32 + ty + j;
      if (it < n_t && il < n_l) tile[ty + j][tx] = p.ops[p.chain.first_slot].ptr[in_base + it * s_t + il * s_l];
    }
    __syncthreads();
    // write: threads run along the last dim (contiguous in the output)
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      int64_t it = tt * 32 + ty + j, il = tl * 32 + tx;
      if (it < n_t && il < n_l) {
        idx[p.tdim] = it;
        idx[last] = il;
        float v = tile[tx][ty + j];
        for (int s = 0; s < p.chain.n; ++s) {
          const ChainStep st = p.chain.steps[s];
          float side = st.imm;
          if (st.slot >= 0) {
            int64_t off = 0;
#pragma unroll
            for (int d = 0; d < kVecRank; ++d)
              if (d < p.rank) off += idx[d] * p.ops[st.slot].stride[d];
            side = p.ops[st.slot].ptr[off];
          }
          v = apply_chain(st.op, v, side);
        }
        int64_t off = 0;
#pragma unroll
        for (int d = 0; d < kVecRank; ++d)
          if (d < p.rank) off += idx[d] * p.ops[p.chain.out_slot].stride[d];
        p.ops[p.chain.out_slot].ptr[off] = v;
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------------------------

static bool chain_slots(const Chain& c, int* slots, int* n) {
  *n = 0;
  if (c.first_slot < 0) return false;
  slots[(*n)++] = c.first_slot;
  for (int s = 0; s < c.n; ++s)
    if (c.steps[s].slot >= 0) slots[(*n)++] = c.steps[s].slot;
  slots[(*n)++] = c.out_slot;
  return true;
}

int choose_elementwise(Plan& plan, PlanKernel& k) {
  (void)plan;
  const kb200_kernel_desc& d = k.desc;
  k.impl = IMPL_EW_GENERIC;
  k.launches = 1;
  k.has_chain = extract_chain(d, &k.chain);
  if (!k.has_chain || d.iter_rank > kVecRank) return KB200_OK;
  int slots[kMaxChain + 2], n_slots;
  if (!chain_slots(k.chain, slots, &n_slots)) return KB200_OK;
  const int last = d.iter_rank - 1;
  const int64_t inner = d.iter_shape[last];
  // vec4: every operand contiguous or constant along the innermost dim, everything 16-byte aligned
  bool vec = inner % 4 == 0 && numel_of(d) / 4 < (int64_t(1) << 31);   // the kernel's indices are 32-bit
  for (int i = 0; i < n_slots && vec; ++i) {
    const DevOperand& o = k.ops[slots[i]];
    const bool is_out = slots[i] == k.chain.out_slot;
    // every element offset (and stride) of the operand fits the kernel's 32-bit arithmetic
    int64_t span = 0;
    for (int dd = 0; dd <= last && vec; ++dd) {
      if (o.stride[dd] < 0) vec = false;
      span += (d.iter_shape[dd] - 1) * o.stride[dd];
    }
    if (span >= (int64_t(1) << 31)) vec = false;
    if (!vec) break;
    if (o.stride[last] == 1) {
      vec = (reinterpret_cast<uintptr_t>(o.ptr) & 15) == 0;
      for (int dd = 0; dd < last && vec; ++dd) vec = o.stride[dd] % 4 == 0;
    } else if (o.stride[last] == 0 && !is_out) {
      // scalar along the row: fine
    } else {
      vec = false;
    }
  }
  if (vec) {
    k.impl = IMPL_EW_CHAIN_VEC4;
    return KB200_OK;
  }
  // transpose: output contiguous along the last dim, first input contiguous along another one
  const DevOperand& in = k.ops[k.chain.first_slot];
  const DevOperand& out = k.ops[k.chain.out_slot];
  if (d.iter_rank >= 2 && out.stride[last] == 1 && in.stride[last] != 1) {
    for (int t = 0; t < last; ++t) {
      if (in.stride[t] == 1 && d.iter_shape[t] >= 8 && inner >= 8) {
        k.impl = IMPL_EW_TRANSPOSE;
        k.x_slot = t;   // reused field: the input's contiguous dim
        return KB200_OK;
      }
    }
  }
  return KB200_OK;
}

int launch_elementwise(const Plan& plan, const PlanKernel& k, cudaStream_t s) {
  const kb200_kernel_desc& d = k.desc;
  const int64_t numel = numel_of(d);
  if (k.impl == IMPL_EW_CHAIN_VEC4) {
    EwChainParams p{};
    const int rank = d.iter_rank;
    for (int i = 0; i < rank; ++i) p.shape[i] = (uint32_t)d.iter_shape[i];
    p.shape[rank - 1] /= 4;
    p.nvec = (uint32_t)(numel / 4);
    for (int o = 0; o < d.n_operands; ++o) {
      p.ptr[o] = k.ops[o].ptr;
      for (int i = 0; i < rank; ++i) p.stride[o][i] = (int32_t)(k.ops[o].stride[i] * (i == rank - 1 ? 4 : 1));
    }
    p.chain = k.chain;
    constexpr int U = 2;
    int64_t blocks = ((int64_t)p.nvec + 256 * U - 1) / (256 * U);
    // beyond the cap every block takes the same number of grid-stride steps (no ragged last wave)
    const int64_t cap = (int64_t)plan.sm_count * 64;
    const int64_t steps = (blocks + cap - 1) / cap;
    const unsigned grid = (unsigned)((blocks + steps - 1) / (steps > 0 ? steps : 1));
    switch (rank) {
      case 1: launch_kernel(plan.pdl, ew_chain_vec4_kernel<1, U>, dim3(grid), dim3(256), 0, s, p); break;
      case 2: launch_kernel(plan.pdl, ew_chain_vec4_kernel<2, U>, dim3(grid), dim3(256), 0, s, p); break;
      case 3: launch_kernel(plan.pdl, ew_chain_vec4_kernel<3, U>, dim3(grid), dim3(256), 0, s, p); break;
      default: launch_kernel(plan.pdl, ew_chain_vec4_kernel<4, U>, dim3(grid), dim3(256), 0, s, p); break;
    }
  } else if (k.impl == IMPL_EW_TRANSPOSE) {
    EwTransposeParams p{};
    p.rank = d.iter_rank;
    p.tdim = k.x_slot;
    p.outer = 1;
    for (int i = 0; i < d.iter_rank; ++i) {
      p.shape[i] = d.iter_shape[i];
      if (i != p.tdim && i != d.iter_rank - 1) p.outer *= d.iter_shape[i];
    }
    for (int o = 0; o < d.n_operands; ++o) p.ops[o] = k.ops[o];
    p.chain = k.chain;
    int64_t tiles = ((p.shape[p.tdim] + 31) / 32) * ((p.shape[p.rank - 1] + 31) / 32) * p.outer;
    int64_t cap = (int64_t)plan.sm_count * 16;
    launch_kernel(plan.pdl, ew_transpose_kernel, dim3((unsigned)(tiles < cap ? tiles : cap)), dim3(256), 0, s, p);
  } else {
    EwParams p{};
    p.rank = d.iter_rank;
    p.n_operands = d.n_operands;
    p.numel = numel;
    for (int i = 0; i < d.iter_rank; ++i) p.shape[i] = d.iter_shape[i];
    for (int o = 0; o < d.n_operands; ++o) p.ops[o] = k.ops[o];
    p.tape = k.tape;
    int64_t blocks = (numel + 255) / 256;
    int64_t cap = (int64_t)plan.sm_count * 8;
    launch_kernel(plan.pdl, ew_generic_kernel, dim3((unsigned)(blocks < cap ? blocks : cap)), dim3(256), 0, s, p);
  }
  KB200_CUDA(cudaGetLastError());
  return KB200_OK;
}

}  // namespace kb200
