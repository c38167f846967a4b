// Which matmul kernel runs a descriptor: exact-FP32 SIMT tiles, the decode GEMV, or tcgen05 tiles.
#include "kb200_internal.h"
#include "matmul.h"

namespace kb200 {

bool tc_eligible(const PlanKernel& k);
int tc_bind(Plan& plan, PlanKernel& k, int kernel_index);
int tc_launch(const Plan& plan, const PlanKernel& k, cudaStream_t s);
void tc_destroy(PlanKernel& k);

int choose_matmul(Plan& plan, PlanKernel& k) {
  (void)plan;
  const kb200_kernel_desc& d = k.desc;
  k.has_chain = extract_chain(d, &k.chain) && k.chain.first_slot == -1;
  k.impl = IMPL_MM_SIMT;
  k.launches = 1;
  const DevOperand& B = k.ops[d.b_slot];
  const int forced = d.cfg[5];   // 0 auto, 1 simt, 2 tc, 3 gemv
  if ((forced == 0 || forced == 3) && k.M == 1 && B.stride[2] == 1 && B.stride[1] % 2 == 0 && B.stride[0] % 2 == 0 &&
      (reinterpret_cast<uintptr_t>(B.ptr) & 7) == 0) {
    k.impl = IMPL_MM_GEMV;
    return KB200_OK;
  }
  if ((forced == 0 || forced == 2) && tc_eligible(k)) k.impl = IMPL_MM_TC;
  if (forced == 2 && k.impl != IMPL_MM_TC)
    return fail(KB200_ERR_UNSUPPORTED, "matmul %s: the tensor-core kernel cannot take these operands", d.name);
  return KB200_OK;
}

int bind_matmul(Plan& plan, PlanKernel& k) {
  if (k.impl != IMPL_MM_TC) return KB200_OK;
  return tc_bind(plan, k, (int)(&k - plan.kernels.data()));
}

int launch_matmul(const Plan& plan, const PlanKernel& k, cudaStream_t s) {
  if (k.impl == IMPL_MM_TC) return tc_launch(plan, k, s);
  return launch_matmul_simt(plan, k, s);
}

void destroy_matmul(PlanKernel& k) { tc_destroy(k); }

}  // namespace kb200
