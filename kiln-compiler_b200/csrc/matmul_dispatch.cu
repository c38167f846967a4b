// Which matmul kernel runs a descriptor: exact-FP32 SIMT tiles, the decode GEMV, or tcgen05 tiles.
#include "kb200_internal.h"
#include "matmul.h"

namespace kb200 {

int choose_matmul(Plan& plan, PlanKernel& k) {
  (void)plan;
  const kb200_kernel_desc& d = k.desc;
  k.has_chain = extract_chain(d, &k.chain) && k.chain.first_slot == -1;
  k.impl = IMPL_MM_SIMT;
  k.launches = 1;
  const DevOperand& B = k.ops[d.b_slot];
  const int forced = d.cfg[5];
  if ((forced == 0 || forced == 3) && k.M == 1 && B.stride[2] == 1 && B.stride[1] % 2 == 0 && B.stride[0] % 2 == 0 &&
      (reinterpret_cast<uintptr_t>(B.ptr) & 7) == 0)
    k.impl = IMPL_MM_GEMV;
  return KB200_OK;
}

int bind_matmul(Plan& plan, PlanKernel& k) {
  (void)plan;
  (void)k;
  return KB200_OK;
}

int launch_matmul(const Plan& plan, const PlanKernel& k, cudaStream_t s) { return launch_matmul_simt(plan, k, s); }

void destroy_matmul(PlanKernel& k) { (void)k; }

}  // namespace kb200
