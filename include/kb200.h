/*
 * kb200.h -- C ABI of the B200-native kernel library behind Kiln's GPU backend.
 *
 * The library replaces what the reference's GPU backend does with generated
 * Triton source: run the fused kernels of one optimised Kiln graph on the
 * device, writing into the single planned arena.  The host side (Python,
 * package kiln_b200) walks the Kiln graph and describes every launch with the
 * plain-old-data structs below; nothing in this interface is a torch type.
 *
 * Threading: a plan is not re-entrant (one arena), exactly like the
 * reference's GPUExecutable (kiln/gpu/runtime.py:135-136).  All functions
 * return 0 on success and a negative kb200_status otherwise; the text of the
 * last failure on the calling thread is returned by kb200_last_error().
 * Nothing here aborts or throws.  Device memory is allocated, and the device
 * synchronised, only while a plan is set up: kb200_plan_create allocates the
 * plan's status word, and kb200_plan_bind allocates the library-owned scratch
 * (in BF16 mode a bf16 mirror of the arena and packed bf16 copies of constant
 * matmul operands; a staging buffer for a fused attention whose output aliases
 * its inputs; in FP32 mode the fused attention's scratch: the operands' tails or
 * the split tiles' partial results), converts the constants (cudaDeviceSynchronize) and reads the
 * attention mask back once (a blocking copy).  kb200_plan_launch and
 * kb200_kernel_launch neither allocate nor synchronise and are therefore
 * capturable into a CUDA graph; kb200_plan_status is a blocking 4-byte copy.
 */
#ifndef KB200_H
#define KB200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KB200_ABI_VERSION 3

#define KB200_MAX_RANK 6      /* iteration dims after the host collapsed contiguous ones */
#define KB200_MAX_OPERANDS 12 /* distinct tensors one fused kernel touches */
#define KB200_MAX_TAPE 96     /* scalar ops of one fused kernel */

typedef enum kb200_status {
  KB200_OK = 0,
  KB200_ERR_ARGUMENT = -1,    /* malformed descriptor, null pointer, rank/slot out of range */
  KB200_ERR_UNSUPPORTED = -2, /* well-formed but no kernel covers it (maps to NotImplementedError) */
  KB200_ERR_BOUNDS = -3,      /* an operand's span leaves the buffer it is bound to */
  KB200_ERR_CUDA = -4,        /* a CUDA call failed; message carries cudaGetErrorString */
  KB200_ERR_UNBOUND = -5,     /* launch before kb200_plan_bind */
  KB200_ERR_DEVICE_WAIT = -6  /* a bounded device-side wait ran out (see kb200_plan_status) */
} kb200_status;

/* Where a tensor lives.  Mirrors the `bases` keys of the reference's Launch
 * (kiln/gpu/codegen.py:106-116): ("arena",) ("const", name) ("input", i) ("output", i). */
typedef enum kb200_base_kind {
  KB200_BASE_ARENA = 0,
  KB200_BASE_CONST = 1,
  KB200_BASE_INPUT = 2,
  KB200_BASE_OUTPUT = 3
} kb200_base_kind;

/* Kernel classes: the four kinds the reference writes (kiln/gpu/codegen.py:532-542). */
typedef enum kb200_kclass {
  KB200_K_ELEMENTWISE = 0, /* codegen.py:284-310; also copies */
  KB200_K_ROW = 1,         /* codegen.py:312-430; LayerNorm, softmax, any row-reduction chain */
  KB200_K_REDUCE = 2,      /* codegen.py:432-482; one reduce over arbitrary dims */
  KB200_K_MATMUL = 3       /* codegen.py:484-530; batched matmul + fused epilogue */
} kb200_kclass;

/* Arithmetic mode of a matmul's operands (accumulation is always FP32).
 * FP32 corresponds to input_precision="ieee", TF32 to "tf32"
 * (codegen.py:515-516); BF16 is a backend-internal mode with no IR dtype.
 * FP32 on the tensor cores is three TF32 products of split operands: within 1e-5 of exact for
 * finite operands, but NOT IEEE for non-finite ones (an infinite operand element yields NaN, see
 * cfg[6] bit 1024 below for the CUDA-core kernel that is). */
typedef enum kb200_precision {
  KB200_PREC_FP32 = 0,
  KB200_PREC_TF32 = 1,
  KB200_PREC_BF16 = 2
} kb200_precision;

/* Scalar op codes of the tape; the table follows _KernelWriter.apply
 * (codegen.py:223-248) and the prelude formulas (codegen.py:53-88). */
typedef enum kb200_opcode {
  KB200_OP_LOAD = 0,   /* a = operand slot */
  KB200_OP_IMM = 1,    /* imm = float32 literal (codegen.py:98-103) */
  KB200_OP_ACC = 2,    /* the matmul accumulator element */
  KB200_OP_ADD = 3, KB200_OP_SUB = 4, KB200_OP_MUL = 5, KB200_OP_DIV = 6,
  KB200_OP_MAX = 7, KB200_OP_MIN = 8,
  KB200_OP_NEG = 9, KB200_OP_RELU = 10, KB200_OP_EXP = 11, KB200_OP_TANH = 12,
  KB200_OP_SIGMOID = 13, KB200_OP_ERF = 14, KB200_OP_GELU_TANH = 15, KB200_OP_GELU_ERF = 16,
  KB200_OP_RSQRT = 17, KB200_OP_SQRT = 18, KB200_OP_COPY = 19,
  KB200_OP_RSUM = 20,  /* keepdim sum over the row (last iteration dim); a = value */
  KB200_OP_RMAX = 21,  /* keepdim max over the row */
  KB200_OP_STORE = 22  /* a = value, b = operand slot */
} kb200_opcode;

/* One tape entry.  Entry i defines value i; `a`/`b` name earlier entries
 * (or, for LOAD/STORE, an operand slot).  `level` is the number of row
 * reductions on the longest path from the kernel's inputs to this value
 * (the pass structure of the chunked row kernel, codegen.py:376-380). */
typedef struct kb200_tape_op {
  int32_t opcode;
  int32_t a;
  int32_t b;
  int32_t level;
  float imm;
} kb200_tape_op;

/* One tensor operand, already aligned to the kernel's iteration space:
 * stride[d] is the element stride along iteration dim d, 0 where the tensor
 * broadcasts (codegen.py:212-216 skips those dims the same way).
 * elem_offset is in float32 elements from the start of the bound buffer;
 * for the arena it already includes the planned byte offset / 4
 * (codegen.py:545-549). */
typedef struct kb200_operand {
  int32_t base_kind;   /* kb200_base_kind */
  int32_t base_index;  /* index into consts / inputs / outputs passed to kb200_plan_bind */
  int64_t elem_offset;
  int64_t stride[KB200_MAX_RANK];
} kb200_operand;

/* Iteration spaces, by class:
 *   ELEMENTWISE  iter_shape = output shape (collapsed); one launch per output.
 *   ROW          iter_shape = row dims..., inner; the reductions run over the last dim.
 *   REDUCE       iter_shape = kept dims..., reduced dims...; n_kept says where they split.
 *   MATMUL       iter_shape = batch, M, N; operands[a_slot].stride = {batch, M, K} strides,
 *                operands[b_slot].stride = {batch, K, N} strides, every other operand
 *                (epilogue inputs, outputs) is aligned to {batch, M, N}.
 */
typedef struct kb200_kernel_desc {
  int32_t kclass;      /* kb200_kclass */
  int32_t precision;   /* kb200_precision; only matmuls look at it */
  int32_t iter_rank;
  int32_t n_kept;      /* REDUCE only */
  int64_t iter_shape[KB200_MAX_RANK];
  int64_t k_extent;    /* MATMUL only: the contraction length K */
  int32_t a_slot;      /* MATMUL only */
  int32_t b_slot;      /* MATMUL only */
  int32_t n_operands;
  int32_t n_tape;
  kb200_operand operands[KB200_MAX_OPERANDS];
  kb200_tape_op tape[KB200_MAX_TAPE];
  /* Tuner configuration, opaque to the reference seam (kiln/api.py:155-162):
   * cfg[0] tile M, cfg[1] tile N, cfg[2] 128-byte K slabs per pipeline stage (1 or 2), cfg[3] pipeline stages,
   * cfg[4] split-K factor, cfg[5] implementation override (0 = library picks),
   * cfg[0] also selects the tensor-core kernel: 0 = library picks, 128 = single-CTA 128-row tiles,
   * 256 = 256-row tiles on SM pairs (cfg[1] then 128 or 256 columns, cfg[2] slabs per step).
   * cfg[6] option bits of the tensor-core matmul (0 = defaults): 512 = two MMA issuers for 64-column
   * single-CTA tiles; 1024 = an FP32-precision matmul runs on the CUDA cores instead of as three TF32
   * products of split operands -- needed when an OPERAND may hold +-inf: the split gives inf - inf = NaN
   * tails, so the product is NaN where IEEE arithmetic gives +-inf (the Python side sets this bit on every
   * matmul when KILN_GPU_FP32_MATMUL=ieee), cfg[7] epilogue stores of the tensor-core matmul (0 = library picks,
   * 1 = ordinary global stores, never bulk tensor stores, 2 = bulk stores but always the
   * transposing lane-per-column epilogue), all 0 = library default. */
  int32_t cfg[8];
  char name[32];       /* the Kiln kernel it comes from, e.g. "k3" (diagnostics only) */
} kb200_kernel_desc;

typedef struct kb200_plan kb200_plan;

/* Library / ABI version; the host side refuses to run against a mismatch. */
int kb200_version(void);

/* Text of the last error on this thread ("" if none).  Never NULL. */
const char* kb200_last_error(void);

/* Builds a launch plan for `n` kernels on CUDA device `device`.
 * Takes the place of kiln.gpu.codegen.generate + load_module
 * (kiln/gpu/codegen.py:601-614, kiln/gpu/runtime.py:58-79): validates every
 * descriptor on the host (ranks, slots, tape references), picks the kernel
 * implementation for each class and returns KB200_ERR_UNSUPPORTED for anything
 * the reference would raise NotImplementedError on.  The descriptors are copied. */
int kb200_plan_create(const kb200_kernel_desc* descs, int n, int device, kb200_plan** out);

/* Binds device buffers.  Takes the place of the `bases` resolution in
 * GPUExecutable._run (kiln/gpu/runtime.py:164-176).  `*_bytes` are the sizes
 * of the buffers; every operand's offset + span is checked against them here,
 * on the host, before anything can run.  Buffers stay owned by the caller and
 * must outlive the launches.  May be called again to re-bind. */
int kb200_plan_bind(kb200_plan* plan, void* arena, uint64_t arena_bytes,
                    void* const* consts, const uint64_t* const_bytes, int n_consts,
                    void* const* inputs, const uint64_t* input_bytes, int n_inputs,
                    void* const* outputs, const uint64_t* output_bytes, int n_outputs);

/* Plan options, set between kb200_plan_create and kb200_plan_bind.
 * KB200_OPT_FUSE_ATTENTION (default 1): when the plan contains the reference's five-kernel
 * attention chain (K^T copy, QK^T * scale + causal mask, softmax, PV, head merge; see
 * tests/models/transformer.py:16-25 of the reference), or the seven-kernel chain of a batch of
 * sequences, run it as one fused kernel (in FP32 precision: with float32 products, behind a small
 * launch that prepares the operands' tails when the tensor cores are used).  The kernel list and
 * arena offsets stay the reference's; the score buffers are then never written.  0 keeps one launch
 * per planned kernel.
 * KB200_OPT_DEPENDENT_LAUNCH (default 1): kernels are enqueued with programmatic stream
 * serialization, so that a kernel's start-up overlaps the tail of the one before it (each kernel
 * waits for its predecessor before it touches global memory).  0 = plain stream order.
 * KB200_OPT_FOLD_OPERAND_COPIES (default 1): where the plan makes a matmul's B operand N-contiguous
 * with a copy kernel (kiln/passes/buffers.py:208-217) that feeds only that matmul, the matmul reads
 * the copy's source as a K-contiguous operand and the copy is not launched.  0 launches every copy.
 * KB200_OPT_CONCURRENCY (default 1): how many plans the caller keeps in flight on this GPU at the
 * same time (a server overlapping requests on several streams).  Only a hint for the tile
 * heuristics, which the reference leaves to its autotuner (kiln/gpu/codegen.py:563-598): with n > 1 a
 * matmul counts on 1/n of the SMs and prefers fewer, wider tiles.  Results do not depend on it.
 * KB200_OPT_ABSORB_ELEMENTWISE (default 1): an elementwise kernel that directly follows a tensor-core
 * matmul and only continues it -- its one arena input is exactly the matmul's output, which nothing
 * else reads -- runs as the tail of the matmul's epilogue, and the matmul writes that kernel's output.
 * This is what the reference's plans contain behind every Linear on a [batch, tokens, d] input: its
 * fusion pass cannot take the activation or the residual add into the matmul's kernel across the
 * reshape between them (kiln/passes/fusion.py:26-35).  0 launches every planned kernel.
 * KB200_OPT_MIRROR_ONLY (default 1, BF16 mode): a LayerNorm or matmul whose output is read only by
 * kernels that take its bf16 mirror (tensor-core matmul operands, the fused attention) does not store
 * the float32 values: that arena region then holds stale data, which no planned kernel reads.  0 stores
 * both, for a caller that inspects intermediate buffers.
 * KB200_OPT_FP32_ATTENTION (default 0, FP32 precision): which kernel runs the fused attention.
 * 0 = by size (the tensor-core kernel, three TF32 products per float32 product, when its work items
 * fill a quarter of the SMs and no matmul of the chain asked for IEEE behaviour on non-finite
 * operands; else the CUDA-core kernel), 1 = always the CUDA-core kernel, 2 = always the tensor cores.
 * KB200_OPT_ATTENTION_SPLIT (default 1): in a launch that leaves SMs idle (one long sequence,
 * KB200_OPT_CONCURRENCY 1) the fused attention shares its long query tiles between two CTAs, which
 * merge their halves through a workspace.  0 keeps every query tile on one CTA. */
typedef enum kb200_option {
  KB200_OPT_FUSE_ATTENTION = 1,
  KB200_OPT_DEPENDENT_LAUNCH = 2,
  KB200_OPT_FOLD_OPERAND_COPIES = 3,
  KB200_OPT_CONCURRENCY = 4,
  KB200_OPT_ABSORB_ELEMENTWISE = 5,
  KB200_OPT_MIRROR_ONLY = 6,
  KB200_OPT_FP32_ATTENTION = 7,
  KB200_OPT_ATTENTION_SPLIT = 8
} kb200_option;
int kb200_plan_set_option(kb200_plan* plan, int option, int value);

/* Enqueues every kernel, in order, on `cuda_stream` (a cudaStream_t).
 * Takes the place of the launch loop GPUExecutable._run
 * (kiln/gpu/runtime.py:164-179).  No synchronisation, no allocation. */
int kb200_plan_launch(kb200_plan* plan, void* cuda_stream);

/* Enqueues kernel `i` alone (profiling, autotuning). */
int kb200_kernel_launch(kb200_plan* plan, int i, void* cuda_stream);

/* Number of device kernel launches kb200_plan_launch enqueues (a Kiln kernel
 * may take more than one: packing an operand, then the matmul). */
int kb200_plan_launch_count(const kb200_plan* plan);

/* Name of the implementation chosen for kernel `i` ("ew_chain_vec4",
 * "row_layernorm_warp", "mm_tcgen05_tf32", ...).  Never NULL for a valid i. */
const char* kb200_kernel_impl(const kb200_plan* plan, int i);

/* Number of fused scalar steps kernel `i` applies per element as bound: the epilogue chain of a
 * matmul (including the steps of an elementwise or row kernel it took over, see
 * KB200_OPT_ABSORB_ELEMENTWISE), the chain of an elementwise kernel, the chain in front of a
 * register-resident row kernel's reductions; 0 for a kernel that launches nothing and for the
 * general tape kernels; -1 for a bad index or an unbound plan.  Introspection only. */
int kb200_kernel_chain_length(const kb200_plan* plan, int i);

/* Reads back the plan's device status word after the caller synchronised:
 * 0 = ok, otherwise KB200_ERR_DEVICE_WAIT with the kernel index in
 * kb200_last_error().  Device-side waits are bounded; when one runs out the
 * kernel records it here and returns normally. */
int kb200_plan_status(kb200_plan* plan);

/* Failure-path self-test (no counterpart in the reference): enqueues a one-warp kernel whose only
 * wait cannot succeed -- an mbarrier that expects two arrivals and receives one, polled a few
 * thousand times, with no copy in flight.  On expiry it records its site in the plan's status word
 * exactly as the tensor-core kernels do and returns normally; after a synchronise,
 * kb200_plan_status then returns KB200_ERR_DEVICE_WAIT (kernel 0xffff, site 0x7f) and the plan, the
 * context and the GPU stay usable.  Nothing traps, faults or spins without bound. */
int kb200_plan_selftest_wait(kb200_plan* plan, void* cuda_stream);

/* Frees the plan and any scratch it owns. */
void kb200_plan_destroy(kb200_plan* plan);

/* C = A * B on the tensor cores with operands rounded to bf16 (FP32 accumulation), for callers
 * that must not allocate.  No counterpart in the reference: it exists for hosts that cannot call
 * cudaMalloc at the point where they need a matmul -- servers that fix their device-memory
 * budget at start-up, latency-critical paths that ban allocation after initialisation, code
 * that cannot afford the device-wide synchronisation an allocation may imply.  The plan interface above obtains the packed bf16 operand
 * copies with cudaMalloc when buffers are bound; here they live in a 16 MiB array that is part
 * of the library image (every GPU that loads the library holds it until the process exits).
 *
 *   a [m, k], b [k, n], c [m, n]: row-major contiguous float32 device buffers, 16-byte aligned;
 *   n >= 64, k >= 64, both multiples of 8.
 *   Limit: 2 * (m*k + k*n) bytes (each operand rounded up to 256) must fit in 16 MiB - 256;
 *   larger shapes are refused with KB200_ERR_ARGUMENT and a message naming both numbers.
 *   status_word: optional device int, zeroed by the caller, that receives a non-zero code if a
 *   bounded device-side wait runs out; pass NULL to use (and have cleared) a word inside the array,
 *   which kb200_matmul_bf16_static_status() reads back.
 *
 * Enqueues three kernels on `cuda_stream` and returns; calls no cudaMalloc, cudaFree or any other
 * allocating routine.  The first call on a device resolves the array's device address
 * (cudaGetSymbolAddress) and raises the kernel's shared-memory limit; make that first call
 * outside any stream capture.  All calls share the one array, which keeps whatever the last call
 * left in it: nothing in it needs to start at zero except the internal status word, which each
 * call clears itself, but two calls that overlap on the GPU (different streams, or graphs
 * replayed concurrently) race on it and corrupt each other's operands. */
int kb200_matmul_bf16_static(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                             int* status_word, void* cuda_stream);

/* After the caller synchronised with the stream: 0, or KB200_ERR_DEVICE_WAIT if a bounded wait of the
 * last kb200_matmul_bf16_static call that passed status_word == NULL ran out on the current device
 * (a blocking 4-byte copy; allocates nothing).  No counterpart in the reference. */
int kb200_matmul_bf16_static_status(void);

#ifdef __cplusplus
}
#endif
#endif /* KB200_H */
