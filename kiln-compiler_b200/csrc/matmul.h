// Shared by the matmul kernels: launch parameters and the fused epilogue.
#pragma once

#include "device_math.cuh"
#include "kb200_internal.h"

namespace kb200 {

struct MatmulParams {
  int64_t batch, M, N, K;
  int a_slot, b_slot, n_operands, has_chain;
  DevOperand ops[KB200_MAX_OPERANDS];   // epilogue operands and outputs are aligned to {batch, M, N}
  Chain chain;                          // valid when has_chain
  DevTape tape;
};

// The epilogue of one accumulator element (kiln/gpu/codegen.py:518-524): the elementwise ops fused
// after the matmul, evaluated on the accumulator, then the store(s).  The chain form keeps the
// running value in a register; any other DAG goes through the general tape.
__device__ __forceinline__ void epilogue_store(const MatmulParams& p, float acc, int64_t b, int64_t m, int64_t n) {
  if (p.has_chain) {
    float v = acc;
    for (int s = 0; s < p.chain.n; ++s) {
      const ChainStep st = p.chain.steps[s];
      float side = st.imm;
      if (st.slot >= 0) {
        const DevOperand& o = p.ops[st.slot];
        side = o.ptr[b * o.stride[0] + m * o.stride[1] + n * o.stride[2]];
      }
      v = apply_chain(st.op, v, side);
    }
    const DevOperand& o = p.ops[p.chain.out_slot];
    o.ptr[b * o.stride[0] + m * o.stride[1] + n * o.stride[2]] = v;
    return;
  }
  float r[KB200_MAX_TAPE];
  for (int t = 0; t < p.tape.n; ++t) {
    const kb200_tape_op op = p.tape.ops[t];
    switch (op.opcode) {
      case KB200_OP_ACC: r[t] = acc; break;
      case KB200_OP_LOAD: {
        const DevOperand& o = p.ops[op.a];
        r[t] = o.ptr[b * o.stride[0] + m * o.stride[1] + n * o.stride[2]];
        break;
      }
      case KB200_OP_IMM: r[t] = op.imm; break;
      case KB200_OP_STORE: {
        const DevOperand& o = p.ops[op.b];
        o.ptr[b * o.stride[0] + m * o.stride[1] + n * o.stride[2]] = r[op.a];
        break;
      }
      default: r[t] = apply_op(op.opcode, r[op.a], r[op.b]); break;
    }
  }
}

void fill_matmul_params(const PlanKernel& k, MatmulParams* p);
int launch_matmul_simt(const Plan& plan, const PlanKernel& k, cudaStream_t s);

}  // namespace kb200
