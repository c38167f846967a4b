// Internal declarations shared by the translation units of libkb200.so.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

#include "kb200.h"

namespace kb200 {

// ---- error reporting (thread-local text behind kb200_last_error) ----
int fail(int status, const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define KB200_CUDA(call)                                   \
  do {                                                     \
    cudaError_t e_ = (call);                               \
    if (e_ != cudaSuccess) return cuda_fail(e_, #call);    \
  } while (0)

// ---- device-side views of a descriptor ----
struct DevOperand {
  float* ptr;  // base + elem_offset, resolved at bind
  int64_t stride[KB200_MAX_RANK];
};

struct DevTape {
  int n;
  kb200_tape_op ops[KB200_MAX_TAPE];
};

// A fused elementwise chain in "running value" form: v = f_i(v, side_i).  Extracted from the
// tape when every value feeds only the next op; lets the vectorised kernels keep v in registers.
enum ChainOp : int {
  CH_ADD = 0, CH_SUB, CH_RSUB, CH_MUL, CH_DIV, CH_RDIV, CH_MAX, CH_MIN,
  CH_NEG, CH_RELU, CH_EXP, CH_TANH, CH_SIGMOID, CH_ERF, CH_GELU_TANH, CH_GELU_ERF, CH_RSQRT, CH_SQRT, CH_COPY,
  // BF16-mode matmul epilogues only (set at bind): tanh through the one-instruction approximation
  CH_TANH_APPROX, CH_GELU_TANH_APPROX
};
constexpr int kMaxChain = 8;
struct ChainStep {
  int op;     // ChainOp
  int slot;   // operand slot of the side input, -1 = immediate, -2 = unary
  float imm;
};
struct Chain {
  int n;
  int first_slot;  // operand slot of the initial value; -1 = the matmul accumulator
  int out_slot;
  ChainStep steps[kMaxChain];
};

// What the library decided for one descriptor.
enum Impl : int {
  IMPL_EW_GENERIC = 0,
  IMPL_EW_CHAIN_VEC4,
  IMPL_EW_TRANSPOSE,
  IMPL_ROW_GENERIC,
  IMPL_ROW_LAYERNORM,
  IMPL_ROW_SOFTMAX,
  IMPL_REDUCE_GENERIC,
  IMPL_MM_SIMT,
  IMPL_MM_GEMV,
  IMPL_MM_TC,
  IMPL_ATTN_FUSED,   // this kernel (the K^T copy) runs the fused attention for itself and the next four
  IMPL_FUSED_AWAY,   // covered by a fused kernel launched earlier: nothing to launch
  IMPL_COUNT
};
const char* impl_name(int impl);

struct PlanKernel {
  kb200_kernel_desc desc;
  int impl = 0;
  int launches = 1;
  DevOperand ops[KB200_MAX_OPERANDS];
  int n_ops = 0;        // operand slots in use: the descriptor's, then the side operands of an absorbed kernel (below)
  DevTape tape;
  Chain chain;          // valid when the impl uses it
  bool has_chain = false;
  // row specialisations
  int x_slot = -1, g_slot = -1, b_slot = -1, out_slot = -1;
  float ln_inv_n = 0.f, ln_eps = 0.f;
  // ... whose input may be a short elementwise chain on the loaded row (x * scale + mask before a
  // softmax, a + b before a LayerNorm), and that value may itself be an output of the kernel
  Chain row_pre;          // steps applied to x_slot's row before the reductions (n == 0: none)
  int pre_out_slot = -1;  // operand that receives the chain's value, or -1
  // matmul
  int64_t batch = 1, M = 0, N = 0, K = 0;
  void* tc = nullptr;   // tensor-core state (tensor maps, packed operands), owned by matmul_tc.cu
  void* attn = nullptr; // fused-attention state, owned by attention.cu
  // BF16 mode: a producer may also write its output, rounded to bf16, into the mirror of the arena
  // (same element offsets) so that the matmul that consumes it needs no conversion pass.
  void* shadow_out = nullptr;     // producer side: mirror address of this kernel's (single) output, or null
  const void* a_shadow = nullptr; // consumer side: mirror address of operand A / B, or null (convert per launch)
  const void* b_shadow = nullptr;
  bool mirror_only = false;       // producer side: every reader of the output takes the mirror, the float32 store is dropped
  // An elementwise kernel that only continues the matmul in front of it (the activation or the residual
  // add behind a Linear on a [batch, tokens, d] input, which the reference's fusion pass cannot put into
  // the matmul's kernel because a reshape sits between them, kiln/passes/fusion.py:26-35) runs as the
  // tail of that matmul's epilogue chain: the matmul writes the elementwise kernel's output.
  int absorbed_by = -1;           // on the elementwise kernel: index of the matmul that runs it
};

struct Plan {
  int device = 0;
  int sm_count = 148;
  bool bound = false;
  std::vector<PlanKernel> kernels;
  int* d_status = nullptr;       // device status word for bounded waits
  bool fuse_attention = true;    // replace the five-kernel attention chain by the fused kernel when it matches
  int fp32_attention = 0;        // FP32 precision: 0 = pick the fused attention kernel by size, 1 = CUDA cores, 2 = tensor cores
  bool attention_split = true;   // share long query tiles between two CTAs when a launch would leave SMs idle
  bool fold_copies = true;       // a matmul reads a K-contiguous B at its source; the plan's transposing copy is not launched
  bool pdl = true;               // programmatic dependent launch: a kernel's start-up overlaps its predecessor's tail
  bool absorb_elementwise = true; // a tensor-core matmul also runs the elementwise kernel that only continues it
  bool mirror_only = true;       // BF16 mode: an output that only mirror readers consume is not stored as float32
  int concurrency = 1;           // plans the caller keeps in flight on this GPU at once (tile heuristics assume their share of the SMs)
  void* arena16 = nullptr;       // bf16 mirror of the arena (library-owned, only when some matmul reads it)
  uint64_t arena16_bytes = 0;
  // bound buffers (for re-validation and the tensor-core path)
  float* arena = nullptr;
  uint64_t arena_bytes = 0;
  std::vector<float*> consts, inputs, outputs;
  std::vector<uint64_t> const_bytes, input_bytes, output_bytes;
};

// ---- tape analysis (host) ----
bool extract_chain(const kb200_kernel_desc& d, Chain* out);
bool match_layernorm(const kb200_kernel_desc& d, PlanKernel* k);
bool match_softmax(const kb200_kernel_desc& d, PlanKernel* k);
constexpr int kMaxRowPre = 4;   // chain steps in front of a register-resident row kernel

// ---- per-class entry points ----
int choose_elementwise(Plan& plan, PlanKernel& k);
int launch_elementwise(const Plan& plan, const PlanKernel& k, cudaStream_t s);
int choose_row(Plan& plan, PlanKernel& k);
int launch_row(const Plan& plan, const PlanKernel& k, cudaStream_t s);
int choose_reduce(Plan& plan, PlanKernel& k);
int launch_reduce(const Plan& plan, const PlanKernel& k, cudaStream_t s);
int choose_matmul(Plan& plan, PlanKernel& k);
int bind_matmul(Plan& plan, PlanKernel& k);      // after pointers are resolved
bool matmul_wants_bf16_operands(const PlanKernel& k);
void attention_set_shadow(PlanKernel& k, void* shadow_out);
bool attention_operand_span(const PlanKernel& k, const float** lo, const float** hi);
void attention_elide_copy(Plan& plan, size_t first);
bool attention_use_mirror(PlanKernel& k, const float* arena_base, const void* mirror_base);
const DevOperand* attention_output(const Plan& plan, size_t first, int64_t* elems);
int launch_matmul(const Plan& plan, const PlanKernel& k, cudaStream_t s);
void destroy_matmul(PlanKernel& k);
int attention_try_fuse(Plan& plan, size_t first);    // plan kernels replaced from `first` on: 5, 7 or 0
int attention_chain_length(const PlanKernel& k);
bool attention_wants_bf16(const PlanKernel& k);
bool attention_reads_mirror(const PlanKernel& k);
bool tc_eligible(const PlanKernel& k);
int attention_launch(const Plan& plan, const PlanKernel& k, cudaStream_t s);
void attention_destroy(PlanKernel& k);
void attention_reset_arrivals(PlanKernel& k);    // after a reported wait error: clear the split tiles' arrival counters

// Every kernel of the library is launched through this: with programmatic stream serialization the
// next kernel in the stream may start (barrier set-up, TMEM allocation, descriptor prefetch) while
// this one is still running; it touches global memory only after pdl_wait() below, which returns
// once the preceding grid has completed and its writes are visible.  Without the attribute (plan
// option off) the two device calls are no-ops.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(bool pdl, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
#endif

inline int64_t numel_of(const kb200_kernel_desc& d) {
  int64_t n = 1;
  for (int i = 0; i < d.iter_rank; ++i) n *= d.iter_shape[i];
  return n;
}

}  // namespace kb200
