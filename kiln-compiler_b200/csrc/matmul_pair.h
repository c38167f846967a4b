// The CTA-pair tensor-core matmul (matmul_pair.cu): 256-row tiles computed by two SMs with
// tcgen05.mma.cta_group::2.  matmul_tc.cu prepares the operands (bf16 mirrors, packed constants,
// per-launch conversions) for both tensor-core kernels and hands the tile work to this one when
// the problem has more than 128 rows and the epilogue is one the pair kernel covers.
#pragma once

#include "kb200_internal.h"

namespace kb200 {

struct PairOperands {
  bool bf16;                 // operands are bf16 (kind::f16), else float32 read as TF32
  const void* a_base;        // [batch, M, K], K contiguous
  int64_t a_row, a_batch;    // strides in elements
  const void* b_base;        // [batch, K, N] N contiguous, or (b_kmajor) [batch, N, K] K contiguous
  int64_t b_row, b_batch;
  bool b_kmajor;
};

// Shape, layout and epilogue tests that need no device pointers beyond those already resolved in `k`.
bool pair_eligible(const Plan& plan, const PlanKernel& k);
// Builds tensor maps and launch parameters.  *state stays null when the kernel declines (the caller
// then uses the single-CTA kernel); a non-zero return is an error.
int pair_bind(Plan& plan, PlanKernel& k, int kernel_index, const PairOperands& ops, void** state);
int pair_launch(const Plan& plan, const void* state, cudaStream_t s);
void pair_destroy(void* state);

}  // namespace kb200
