// Fused causal attention for sm_100a: QK^T -> online softmax -> PV in one kernel on the tensor cores.
//
// The fusion pass of the reference leaves attention as five kernels (tests/models/transformer.py:16-25
// after kiln/passes/fusion.py and buffers.py): a copy that makes K^T N-contiguous, a batched matmul
// with the scale + mask epilogue that writes [H, T, T] scores, a softmax row kernel over them, a
// batched matmul with V, and a copy that merges the heads.  The reference lists "no fused attention"
// as a limitation (README.md:185): the scores cross HBM twice.  When the plan contains exactly that
// chain and the mask is the causal one, a fused kernel replaces the five launches: it reads Q, K and
// V as strided views of the QKV projection's output and writes the merged-heads buffer, the only
// value of the chain that is live afterwards.  The plan itself (kernel list, arena offsets) is
// untouched; the score buffers are simply never written.  Two kernels: `attention_kernel` on the tensor
// cores -- for the TF32 and BF16 matmul modes (described next) and, with its EXACT parameter, for FP32
// mode (the same structure with three TF32 MMAs per product) -- and `attention_fp32_kernel` for short
// sequences in FP32 mode (CUDA cores).
//
// Persistent CTAs (one per SM) walk the (sequence, head, 128-query tile) work items, heaviest first, in
// steps of the grid size: barrier set-up, the TMEM allocation and the latency of an item's first
// loads are paid once per CTA or hidden under the previous item's tail, not once per item.  Ring
// slots and barrier phases run on a tile counter that continues across items.  320 threads in three roles:
//   warp 0      TMA producer: Q once, then K and V tiles of 128 keys through 2-deep rings.
//   warp 1      MMA issuer: S = Q K^T (operands in shared memory, TF32) into one of two S buffers in
//               TMEM; O_part = P V with P read from TMEM (written there by the softmax warps).
//   warps 2..9  softmax.  Two threads share a query row (TMEM lane); thread g takes keys g*64 ..
//               g*64+63 of every tile.  One online-softmax state per row: each tile the two exchange
//               the maxima of their halves through shared memory (a 64-thread barrier per lane
//               quadrant), scale, mask the diagonal tile, store P back over S in TMEM; one P V of
//               128 keys accumulates into one O_part (double buffered, folded into the running
//               output one tile late, so the P V of tile j runs under the softmax of tile j+1);
//               thread g folds, normalises and stores head dims g*32 .. g*32+31 through a staging
//               slot per warp and bulk tensor stores.
// Causal tiles above the diagonal are skipped.  Every mbarrier wait is bounded (see matmul_tc.cu).
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <utility>
#include <vector>

#include "device_math.cuh"
#include "kb200_internal.h"
#include "tc_common.cuh"
#include "tc_epilogue.cuh"

namespace kb200 {

namespace {

using namespace tc;

constexpr int kRows = 128;                   // queries per CTA and keys per tile
constexpr int kHeadDim = 64;
constexpr int kSlab = kRows * 128;           // one [128 rows x 128 bytes] swizzled slab
constexpr int kAttnThreads = 64 + 256;
constexpr int kExchangeBytes = 2 * (2 * 2 * kRows * 4);   // the pairs' maxima (two tile parities) and row sums (two item parities)
constexpr int kStageBytes = 4096 + 2048;      // a warp's output rows: 32 x 32 float32 and their bf16 copy
// Q + 2 x K + 2 x V tiles (two 16 KB slabs each in float32, one in bf16), the two merge buffers, alignment slack
constexpr int attn_smem(bool bf16) { return 5 * (bf16 ? 1 : 2) * kSlab + kExchangeBytes + 8 * kStageBytes + 1024; }
// FP32 mode on the tensor cores: Q, K, V once each with their tails (4 slabs per operand), the exchange area, slack
constexpr int kExactSmemBytes = 3 * 4 * kSlab + kExchangeBytes + 1024;

struct AttnParams {
  int T, H, q_tiles;
  int B;                     // sequences in the graph (1 for the two-dimensional block); rows of Q, K, V and of the output are b * T + t
  float scale_log2;          // softmax scale times log2(e): exponentials are taken in base 2
  float* out;                // [T, H * 64] merged heads
  int64_t out_row_stride;
  __nv_bfloat16* out16;      // optional bf16 copy of the merged heads, row stride H * 64, or null
  int64_t out16_row_stride;
  uint32_t idesc_qk, idesc_pv;
  int kernel_index;
  int* status;
  int split_from;            // query tiles from this one on are shared by two CTAs (q_tiles: none)
  float* partial;            // [split tile][2 halves][128 x 64 unnormalised output | 128 maxima | 128 sums]
  int* arrivals;             // [split tile][4 lane quadrants], zero between launches
  const unsigned short* order;   // with split tiles: (query tile << 1 | half) of the q_tiles + split tiles entries, heaviest first
};
constexpr int kPartialFloats = kRows * kHeadDim + 2 * kRows;

constexpr int kFTile = 64;                 // queries per CTA and keys per tile
constexpr int kFPitch = 68;                // floats per shared-memory row of Q, K and P (16-byte aligned, rows 4 banks apart)
constexpr int kFThreads = 128;
constexpr int kFRows = 8;                  // query rows per thread (64 rows over 8 thread rows)
constexpr int kFSmemBytes = (4 * kFTile * kFPitch + 2 * kFTile * kHeadDim) * 4;   // Q, P, two K tiles | two V tiles

struct AttnF32Params {
  const float* q;
  const float* k;
  const float* v;
  int64_t row_stride;        // floats between consecutive tokens of the Q / K / V views
  float* out;                // [B * T, H * 64] merged heads
  int64_t out_row_stride;
  int T, H, B, q_tiles;      // q_tiles = T / 64
  float scale_log2;
  // Query tiles from `split_from` on (the long causal prefixes) are worked on by two CTAs, one per half
  // of the key tiles; each leaves its unnormalised output and softmax state in `partial`, and the one
  // that finishes second (a counter per tile in `arrivals`) merges the two and writes the rows.
  int split_from;
  float* partial;            // [split item][2 halves][64 x 64 output | 64 maxima | 64 sums]
  int* arrivals;             // [split item], zero between launches
};
constexpr int kFPartialFloats = kFTile * kHeadDim + 2 * kFTile;

struct AttnState {
  CUtensorMap map_q, map_k, map_v;
  CUtensorMap map_out, map_out16;   // bulk-store maps of the merged heads [B * T, H * 64] and of their bf16 copy
  // BF16 mode: Q, K and V are read from the bf16 mirror of the QKV projection's output (set after the
  // mirror is allocated); the kernel then runs its matmuls with bf16 operands and P rounded to bf16.
  bool bf16 = false;
  const float* q_ptr = nullptr;
  const float* k_ptr = nullptr;
  const float* v_ptr = nullptr;
  int64_t row_stride = 0;
  AttnParams params;
  dim3 grid;
  // When the planner put the merged-heads buffer over the (by then dead) QKV buffer, the fused
  // kernel cannot write it while other CTAs still read Q, K and V: it writes here, a copy follows.
  const DevOperand* y = nullptr;   // the head-merge kernel's output operand (the chain's only live result)
  int64_t y_elems = 0;
  float* staged_out = nullptr;
  float* final_out = nullptr;
  int64_t out_elems = 0;
  int chain = 5;                   // plan kernels this launch stands for: 5 (one sequence) or 7 (a batch of sequences)
  bool wants_bf16 = false;         // the chain's matmuls are in BF16 mode
  bool exact = false;              // FP32 mode: float32 products, on the tensor cores (three TF32 MMAs each) or on the FMA pipes
  bool exact_tc = false;           // ... on the tensor cores (enough work items to fill the GPU), else the CUDA-core kernel
  AttnF32Params f32;
  void* f32_scratch = nullptr;     // CUDA-core kernel: the split tiles' partial results and arrival counters
  void* split_scratch = nullptr;   // tensor-core kernels: the same for their split tiles
  CUtensorMap map_qt, map_kt, map_vt;   // tensor-core FP32 kernel: Q, K, V views of the tails buffer
  float* tails = nullptr;          // tails (x minus its 19 leading bits) of the span of the QKV buffer the views cover
  const float* span_lo = nullptr;
  int64_t span_n4 = 0;
};

// tails[i] = src[i] minus its 19 leading bits (what a TF32 operand keeps): the second terms of the
// split products of the FP32-mode tensor-core attention.
__global__ void __launch_bounds__(256) tails_kernel(const float4* __restrict__ src, float4* __restrict__ dst, int64_t n4) {
  pdl_wait();                 // the producer of Q, K and V has completed
  pdl_launch_dependents();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    const float4 v = src[i];
    float4 t;
    t.x = v.x - __uint_as_float(__float_as_uint(v.x) & 0xFFFFE000u);
    t.y = v.y - __uint_as_float(__float_as_uint(v.y) & 0xFFFFE000u);
    t.z = v.z - __uint_as_float(__float_as_uint(v.z) & 0xFFFFE000u);
    t.w = v.w - __uint_as_float(__float_as_uint(v.w) & 0xFFFFE000u);
    dst[i] = t;
  }
}

__global__ void __launch_bounds__(256) copy_rows_kernel(const float4* __restrict__ src, float4* __restrict__ dst, int64_t n4) {
  pdl_wait();                 // the producer of this kernel's inputs has completed
  pdl_launch_dependents();    // the next kernel may begin its start-up
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) dst[i] = src[i];
}

// 2^x for x <= 0 through the bare special-function instruction (exp2f adds a range fix-up for
// denormal results, which a probability does not need; the softmax is bound by this pipe).
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Scores of one 32-column block -> probabilities, in place; returns their sum.  `first_col` is the
// block's first key relative to the query tile's first row (only used on the diagonal tile).
template <bool DIAGONAL>
__device__ __forceinline__ float probabilities32(float (&v)[32], float scale_log2, float m_use, int first_col, int row) {
  const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(-m_use, -m_use);
  float2 sum2 = make_float2(0.0f, 0.0f);
#pragma unroll
  for (int i = 0; i < 32; i += 2) {
    const float2 t = ffma2(make_float2(v[i], v[i + 1]), scale2, shift2);     // two exponents per instruction
    float2 pr = make_float2(ex2(t.x), ex2(t.y));
    if (DIAGONAL && first_col + i > row) pr.x = 0.0f;
    if (DIAGONAL && first_col + i + 1 > row) pr.y = 0.0f;
    v[i] = pr.x;
    v[i + 1] = pr.y;
    sum2 = fadd2(sum2, pr);
  }
  return sum2.x + sum2.y;
}
template <bool DIAGONAL>
__device__ __forceinline__ float row_max32(const float (&v)[32], float m, int first_col, int row) {
  if (DIAGONAL) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (first_col + i <= row) m = fmaxf(m, v[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 32; i += 2) m = fmax3(m, v[i], v[i + 1]);
  }
  return m;
}

// ---------------------------------------------------------------------------------------------
// FP32 mode: the same fusion on the CUDA cores.
//
// In FP32 mode (the reference's allow_tf32=False, kiln/gpu/codegen.py:515) the products must be
// float32 products, which the tensor cores only give through three TF32 MMAs on split operands; with
// Q, K, V and P all split that does not fit one CTA's shared and tensor memory next to the softmax.
// This kernel keeps the arithmetic on the FMA pipes instead: one CTA per (sequence, head, 64 queries
// [, half of the keys]), key tiles of 64, 128 threads as 8 x 16, each with an 8 x 4 block of the
// scores (rows ty + 8 i, keys tx + 16 j: every quarter-warp load of K then covers all 32 banks) and
// an 8 x 4 block of the output (rows ty + 8 i, dims 4 tx ..).  What bounds such a kernel is the
// shared-memory-to-register path (128 bytes per clock and SM, whatever is broadcast): a 4 x 4 block
// per thread loads half a float per multiply-add and stopped at 53 % of the FMA pipe; 8 x 4 loads
// 0.375.  A row's 64 scores live in the 16 lanes of one half-warp: maxima and sums go through
// shuffles, and the probabilities a half-warp writes to shared memory are read back by that
// half-warp only.  Online softmax in base 2 with Q pre-multiplied by scale * log2(e); causal tiles
// above the diagonal are skipped; K / V tiles arrive through a two-deep cp.async ring.  The scores
// never leave the SM.
__device__ __forceinline__ void cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}

__global__ void __launch_bounds__(kFThreads, 2) attention_fp32_kernel(const __grid_constant__ AttnF32Params p) {
  extern __shared__ __align__(16) float fsm[];
  float* const Qs = fsm;                               // [64 queries][68]
  float* const Ps = Qs + kFTile * kFPitch;             // [64 queries][68] probabilities of the current tile
  float* const Ks = Ps + kFTile * kFPitch;             // 2 x [64 keys][68]
  float* const Vs = Ks + 2 * kFTile * kFPitch;         // 2 x [64 keys][64]
  pdl_wait();                 // Q, K and V are the previous kernel's output
  pdl_launch_dependents();
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  // work item: the halves of the split query tiles first (longest causal prefixes first), then the rest
  const int w = blockIdx.x;
  const int h = w % p.H;
  const int seq = (w / p.H) % p.B;
  const int v = w / (p.H * p.B);
  const int n_split = p.q_tiles - p.split_from;
  const bool split = v < 2 * n_split;
  const int qt = split ? p.q_tiles - 1 - (v >> 1) : p.split_from - 1 - (v - 2 * n_split);
  const int half = split ? (v & 1) : 0;
  const int j_begin = split && half ? (qt + 1) >> 1 : 0;            // key tiles [j_begin, j_end)
  const int j_end = split && !half ? (qt + 1) >> 1 : qt + 1;
  const int64_t row0 = (int64_t)seq * p.T;
  const int64_t rs = p.row_stride;
  const float* const qg = p.q + (row0 + (int64_t)qt * kFTile) * rs + h * kHeadDim;
  const float* const kg = p.k + row0 * rs + h * kHeadDim;
  const float* const vg = p.v + row0 * rs + h * kHeadDim;
  // a 64 x 64 tile is 1024 float4: thread t moves float4 t, t + 128, ... (row = index / 16)
  const int ld_r = tid >> 4, ld_c = (tid & 15) * 4;
  auto fetch = [&](int j) {
    float* const kd = Ks + (j & 1) * kFTile * kFPitch;
    float* const vd = Vs + (j & 1) * kFTile * kHeadDim;
    const int64_t first = (int64_t)j * kFTile;
#pragma unroll
    for (int i = 0; i < kFRows; ++i) {
      cp_async16(kd + (ld_r + 8 * i) * kFPitch + ld_c, kg + (first + ld_r + 8 * i) * rs + ld_c);
      cp_async16(vd + (ld_r + 8 * i) * kHeadDim + ld_c, vg + (first + ld_r + 8 * i) * rs + ld_c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch(j_begin);
#pragma unroll
  for (int i = 0; i < kFRows; ++i) {
    float4 q4 = __ldg(reinterpret_cast<const float4*>(qg + (int64_t)(ld_r + 8 * i) * rs + ld_c));
    q4.x *= p.scale_log2; q4.y *= p.scale_log2; q4.z *= p.scale_log2; q4.w *= p.scale_log2;
    *reinterpret_cast<float4*>(Qs + (ld_r + 8 * i) * kFPitch + ld_c) = q4;
  }
  float2 o2[kFRows][2];        // dims (4 tx, 4 tx + 1) and (4 tx + 2, 4 tx + 3)
  float m_run[kFRows], l_run[kFRows];
#pragma unroll
  for (int i = 0; i < kFRows; ++i) {
    m_run[i] = -CUDART_INF_F;
    l_run[i] = 0.0f;
    o2[i][0] = o2[i][1] = make_float2(0.0f, 0.0f);
  }
  for (int j = j_begin; j < j_end; ++j) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();          // tile j has landed for everyone (Q too), and everyone is done with tile j - 1
    if (j + 1 < j_end) fetch(j + 1);
    const float* const Kt = Ks + (j & 1) * kFTile * kFPitch;
    const float* const Vt = Vs + (j & 1) * kFTile * kHeadDim;
    // ---- scores: s[i][jj] = q[ty + 8 i] . k[tx + 16 jj] ----
    // Packed multiply-adds (two per instruction): the even and the odd head dims of a product are
    // summed apart -- both operand pairs are then halves of the 128-bit loads as they stand -- and
    // added at the end.
    float2 s2[kFRows][4];
#pragma unroll
    for (int i = 0; i < kFRows; ++i)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) s2[i][jj] = make_float2(0.0f, 0.0f);
#pragma unroll 2
    for (int kk = 0; kk < kHeadDim; kk += 4) {
      float4 b[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) b[jj] = *reinterpret_cast<const float4*>(Kt + (tx + 16 * jj) * kFPitch + kk);
#pragma unroll
      for (int i = 0; i < kFRows; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(Qs + (ty + 8 * i) * kFPitch + kk);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          s2[i][jj] = ffma2(make_float2(a.x, a.y), make_float2(b[jj].x, b[jj].y), s2[i][jj]);
          s2[i][jj] = ffma2(make_float2(a.z, a.w), make_float2(b[jj].z, b[jj].w), s2[i][jj]);
        }
      }
    }
    float s[kFRows][4];
#pragma unroll
    for (int i = 0; i < kFRows; ++i)
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) s[i][jj] = s2[i][jj].x + s2[i][jj].y;
    if (j == qt) {            // the diagonal tile: keys after the query are masked
#pragma unroll
      for (int i = 0; i < kFRows; ++i)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
          if (tx + 16 * jj > ty + 8 * i) s[i][jj] = -CUDART_INF_F;
    }
    // ---- online softmax, one row per half-warp ----
#pragma unroll
    for (int i = 0; i < kFRows; ++i) {
      float mx = fmaxf(fmaxf(s[i][0], s[i][1]), fmaxf(s[i][2], s[i][3]));
#pragma unroll
      for (int d = 8; d >= 1; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
      const float m_new = fmaxf(m_run[i], mx);       // finite: the first key of a tile is never masked
      const float alpha = exp2f(m_run[i] - m_new);
      m_run[i] = m_new;
      float sum = 0.0f;
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const float pr = exp2f(s[i][jj] - m_new);
        sum += pr;
        Ps[(ty + 8 * i) * kFPitch + tx + 16 * jj] = pr;
      }
#pragma unroll
      for (int d = 8; d >= 1; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
      l_run[i] = fmaf(l_run[i], alpha, sum);
      o2[i][0] = fmul2(o2[i][0], make_float2(alpha, alpha));
      o2[i][1] = fmul2(o2[i][1], make_float2(alpha, alpha));
    }
    __syncwarp();             // a row's probabilities are written and read by the same half-warp
    // ---- o[i][d] += sum over keys of P[ty + 8 i][key] * V[key][4 tx + d] ----
#pragma unroll 2
    for (int key = 0; key < kFTile; key += 4) {
      float4 b[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) b[q] = *reinterpret_cast<const float4*>(Vt + (key + q) * kHeadDim + 4 * tx);
#pragma unroll
      for (int i = 0; i < kFRows; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(Ps + (ty + 8 * i) * kFPitch + key);
        // dims (0, 1) and (2, 3) as pairs; a probability is duplicated into both halves of its operand
        o2[i][0] = ffma2(make_float2(a.x, a.x), make_float2(b[0].x, b[0].y), o2[i][0]);
        o2[i][1] = ffma2(make_float2(a.x, a.x), make_float2(b[0].z, b[0].w), o2[i][1]);
        o2[i][0] = ffma2(make_float2(a.y, a.y), make_float2(b[1].x, b[1].y), o2[i][0]);
        o2[i][1] = ffma2(make_float2(a.y, a.y), make_float2(b[1].z, b[1].w), o2[i][1]);
        o2[i][0] = ffma2(make_float2(a.z, a.z), make_float2(b[2].x, b[2].y), o2[i][0]);
        o2[i][1] = ffma2(make_float2(a.z, a.z), make_float2(b[2].z, b[2].w), o2[i][1]);
        o2[i][0] = ffma2(make_float2(a.w, a.w), make_float2(b[3].x, b[3].y), o2[i][0]);
        o2[i][1] = ffma2(make_float2(a.w, a.w), make_float2(b[3].z, b[3].w), o2[i][1]);
      }
    }
    __syncwarp();             // before the next tile's probabilities overwrite these
  }
  float o[kFRows][4];
#pragma unroll
  for (int i = 0; i < kFRows; ++i) {
    o[i][0] = o2[i][0].x; o[i][1] = o2[i][0].y; o[i][2] = o2[i][1].x; o[i][3] = o2[i][1].y;
  }
  if (split) {
    // Leave this half's state in the workspace; the CTA that arrives second merges.  No CTA waits
    // for another: whoever is first just leaves.
    const int item = (seq * p.H + h) * n_split + (qt - p.split_from);
    float* const mine = p.partial + ((size_t)item * 2 + half) * kFPartialFloats;
    const float* const other = p.partial + ((size_t)item * 2 + (half ^ 1)) * kFPartialFloats;
#pragma unroll
    for (int i = 0; i < kFRows; ++i) {
      __stcg(reinterpret_cast<float4*>(mine + (ty + 8 * i) * kHeadDim + 4 * tx), make_float4(o[i][0], o[i][1], o[i][2], o[i][3]));
      if (tx == 0) {
        __stcg(mine + kFTile * kHeadDim + ty + 8 * i, m_run[i]);
        __stcg(mine + kFTile * kHeadDim + kFTile + ty + 8 * i, l_run[i]);
      }
    }
    __threadfence();
    __shared__ int second;
    __syncthreads();
    if (tid == 0) {
      second = atomicAdd(p.arrivals + item, 1);
      __threadfence();
    }
    __syncthreads();
    if (!second) return;
    if (tid == 0) p.arrivals[item] = 0;            // for the next launch
#pragma unroll
    for (int i = 0; i < kFRows; ++i) {
      const float m2 = __ldcg(other + kFTile * kHeadDim + ty + 8 * i);
      const float l2 = __ldcg(other + kFTile * kHeadDim + kFTile + ty + 8 * i);
      const float4 o2 = __ldcg(reinterpret_cast<const float4*>(other + (ty + 8 * i) * kHeadDim + 4 * tx));
      const float m = fmaxf(m_run[i], m2);
      const float a1 = exp2f(m_run[i] - m), a2 = exp2f(m2 - m);
      // products rounded one by one and then added (no fused multiply-add): symmetric in the two
      // halves, so the bits do not depend on which CTA merges
      l_run[i] = __fadd_rn(__fmul_rn(l_run[i], a1), __fmul_rn(l2, a2));
      o[i][0] = __fadd_rn(__fmul_rn(o[i][0], a1), __fmul_rn(o2.x, a2));
      o[i][1] = __fadd_rn(__fmul_rn(o[i][1], a1), __fmul_rn(o2.y, a2));
      o[i][2] = __fadd_rn(__fmul_rn(o[i][2], a1), __fmul_rn(o2.z, a2));
      o[i][3] = __fadd_rn(__fmul_rn(o[i][3], a1), __fmul_rn(o2.w, a2));
    }
  }
  float* const og = p.out + (row0 + (int64_t)qt * kFTile) * p.out_row_stride + h * kHeadDim + 4 * tx;
#pragma unroll
  for (int i = 0; i < kFRows; ++i) {
    const float inv = 1.0f / l_run[i];
    *reinterpret_cast<float4*>(og + (int64_t)(ty + 8 * i) * p.out_row_stride) =
        make_float4(o[i][0] * inv, o[i][1] * inv, o[i][2] * inv, o[i][3] * inv);
  }
}

// EXACT (FP32 mode on the tensor cores, never with BF16): float32 products from three TF32 MMAs each
// (x = head + tail, head the 19 leading bits the tensor core reads anyway: x y ~ head head + head tail
// + tail head).  The tails of Q, K and V come from a copy of the QKV buffer that a small kernel
// fills in front of this one (`tails_kernel`), through tensor maps of their own into the second
// half of every operand buffer; the softmax threads write the probabilities' tails into tensor
// memory next to the probabilities.  Differences in structure, all for space: K and V have one
// buffer each instead of a ring of two (heads + tails of Q, K, V fill 192 KB; the next tile's loads
// run under the softmax, which is the long pole), the tails of P have one buffer (a thread folds the
// previous tile's O_part -- whose completion says its P V has read them -- before it writes the
// next), and the output rows leave by ordinary stores (no staging slots).
template <bool BF16, bool SPLIT, bool EXACT>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_out,
                 const __grid_constant__ CUtensorMap map_out16, const __grid_constant__ CUtensorMap map_qt,
                 const __grid_constant__ CUtensorMap map_kt, const __grid_constant__ CUtensorMap map_vt,
                 const __grid_constant__ AttnParams p) {
  static_assert(!(BF16 && EXACT), "the FP32 mode has float32 operands");
  // a [128 rows x 64 dims] operand tile is two 128-byte-wide slabs in float32, one in bf16;
  // EXACT: an operand buffer holds the tile and, behind it, its tails
  constexpr int kTileSlabs = BF16 ? 1 : 2;
  constexpr int kTileBytes = kTileSlabs * kSlab;
  constexpr int kOpBytes = 2 * kTileBytes;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[20];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int arrived[4];                  // split items: was this lane quadrant's half the second to arrive?

#ifdef KB200_TRACE
  __shared__ long long trace[4][16];
  __shared__ long long mma_trace[64];
  __shared__ long long marks[4];
  int tm = 0;
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long g;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
    marks[0] = (long long)g;
    marks[1] = clock64();
  }
#define ATTN_STAMP(role, idx) do { if (blockIdx.x == 0 && threadIdx.x == 64 && (idx) < 16) trace[role][idx] = clock64(); } while (0)
#define ATTN_MMA_STAMP(idx) do { if (blockIdx.x == 0 && (idx) < 64) mma_trace[idx] = clock64(); } while (0)
#else
#define ATTN_STAMP(role, idx) do { } while (0)
#define ATTN_MMA_STAMP(idx) do { } while (0)
#endif
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t q_smem = (raw + 1023u) & ~1023u;
  const uint32_t k_smem = q_smem + (EXACT ? kOpBytes : kTileBytes);   // ring of 2 tiles | EXACT: one buffer (tile, then its tails)
  const uint32_t v_smem = k_smem + 2 * kTileBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // bars (EXACT uses only the first of each K / V pair): 0 q_full | 1,2 k_full | 3,4 k_empty | 5,6 v_full | 7,8 v_empty | 9,10 s_full |
  //       11..14 p_full[group][s buffer] | 15..18 o_full[group][o buffer] | 19 q_empty
  const uint32_t q_full = smem_u32(&bars[0]), k_full = smem_u32(&bars[1]), k_empty = smem_u32(&bars[3]);
  const uint32_t v_full = smem_u32(&bars[5]), v_empty = smem_u32(&bars[7]);
  const uint32_t sfull0 = smem_u32(&bars[9]), pfull0 = smem_u32(&bars[11]), ofull0 = smem_u32(&bars[15]);
  const uint32_t q_empty = smem_u32(&bars[19]);

  // work item w -> (head, sequence, query tile): heaviest (longest causal prefix) tiles first, of every sequence
  // Query tiles from p.split_from on (the longest causal prefixes; none when split_from = q_tiles) are
  // TWO items, one per half of their key tiles: each leaves its unnormalised rows and softmax state in
  // a workspace, and the one that arrives second (a counter per tile and lane quadrant) merges them.
  // (SPLIT is a template parameter so that the kernel without split tiles keeps its code: with the
  // choice made at run time the eight-sequence attention took 44.4 instead of 43.4 us.)
  const int n_split = SPLIT ? p.q_tiles - p.split_from : 0;
  const int n_items = p.B * p.H * (p.q_tiles + n_split);
  // This CTA's r-th item (-1: none).  Rounds alternate direction over the CTAs, so that the CTA with the
  // heaviest item of one round takes the lightest of the next (24 key tiles at most per CTA instead of
  // 27 for 8 x 12 x 8 items on 148 CTAs).
  auto nth_item = [&](int r) {
    const int w = r * (int)gridDim.x + ((r & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x);
    return w < n_items ? w : -1;
  };
  struct Item { int h, q0, n_kv, row0, qt, j0, half, slot; bool split; };
  auto item_of = [&](int w) {
    Item it;
    it.h = w % p.H;
    const int seq = (w / p.H) % p.B;
    const int v = w / (p.H * p.B);
    if (!SPLIT) {                                      // heaviest (longest causal prefix) first
      it.qt = p.q_tiles - 1 - v;
      it.half = 0;
    } else {                                           // whole tiles and halves in descending order of their key tiles (host table)
      const unsigned e = __ldg(p.order + v);
      it.qt = (int)(e >> 1);
      it.half = (int)(e & 1);
    }
    it.split = SPLIT && it.qt >= p.split_from;
    it.q0 = it.qt * kRows;
    const int n = it.qt + 1;                           // causal: key tiles 0..qt
    it.j0 = it.split && it.half ? n >> 1 : 0;          // this item's key tiles: j0 .. j0 + n_kv - 1
    it.n_kv = (it.split && !it.half ? n >> 1 : n) - it.j0;
    it.slot = it.split ? (seq * p.H + it.h) * n_split + (it.qt - p.split_from) : 0;
    it.row0 = seq * p.T;                               // this sequence's first row in Q, K, V and the output
    return it;
  };

  if (threadIdx.x == 32) {
    prefetch_tensormap(&map_q);
    prefetch_tensormap(&map_k);
    prefetch_tensormap(&map_v);
    if constexpr (EXACT) {
      prefetch_tensormap(&map_qt);
      prefetch_tensormap(&map_kt);
      prefetch_tensormap(&map_vt);
    } else {
      prefetch_tensormap(&map_out);
      if (p.out16 != nullptr) prefetch_tensormap(&map_out16);
    }
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(k_full + 8 * s, 1);
      mbar_init(k_empty + 8 * s, 1);
      mbar_init(v_full + 8 * s, 1);
      mbar_init(v_empty + 8 * s, 1);
      mbar_init(sfull0 + 8 * s, 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(pfull0 + 8 * i, 128);
      mbar_init(ofull0 + 8 * i, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  // Everything above overlapped the previous kernel's tail; Q, K and V are its output.
  pdl_wait();
  pdl_launch_dependents();
  const uint32_t tmem_base = tmem_base_slot;
  // columns: S0 0..127 | S1 128..255 | O_part[buffer] 256 + buffer * 64 | EXACT: tails of P 384..511
  const uint32_t tmem_o0 = tmem_base + 256;
  [[maybe_unused]] const uint32_t tmem_pt = tmem_base + 384;
  volatile int* abort_ptr = &abort_flag;
  auto give_up = [&](int site) {
    if (!*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | site); *abort_ptr = 1; }
  };

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int t = 0;                                     // key tiles loaded so far, over all items
      bool ok = true;
      for (int ii = 0; ok; ++ii) {
        const int w = nth_item(ii);
        if (w < 0) break;
        const Item it = item_of(w);
        // the Q tile is free once every Q K^T of the previous item has been executed
        if (!mbar_wait(q_empty, (ii & 1) ^ 1, abort_ptr)) { give_up(0x13); break; }
        // EXACT, an operand buffer: the tile's two slabs, then the two slabs of its tails
        [[maybe_unused]] auto load4 = [&](uint32_t dst, const CUtensorMap* heads, const CUtensorMap* tails, uint32_t bar, int first_row) {
          mbar_expect_tx(bar, kOpBytes);
          tma_load_3d(dst, heads, bar, 0, first_row, it.h);
          tma_load_3d(dst + kSlab, heads, bar, 32, first_row, it.h);
          tma_load_3d(dst + kTileBytes, tails, bar, 0, first_row, it.h);
          tma_load_3d(dst + kTileBytes + kSlab, tails, bar, 32, first_row, it.h);
        };
        if constexpr (EXACT) {
          load4(q_smem, &map_q, &map_qt, q_full, it.row0 + it.q0);
        } else {
          mbar_expect_tx(q_full, kTileBytes);
          tma_load_3d(q_smem, &map_q, q_full, 0, it.row0 + it.q0, it.h);
          if (!BF16) tma_load_3d(q_smem + kSlab, &map_q, q_full, 32, it.row0 + it.q0, it.h);
        }
        for (int j = 0; j < it.n_kv; ++j, ++t) {
          if constexpr (EXACT) {
            const uint32_t ph = t & 1;                   // one buffer: the phase alternates with every tile
            if (!mbar_wait(k_empty, ph ^ 1, abort_ptr)) { give_up(0x11); ok = false; break; }
            load4(k_smem, &map_k, &map_kt, k_full, it.row0 + (it.j0 + j) * kRows);
            if (!mbar_wait(v_empty, ph ^ 1, abort_ptr)) { give_up(0x12); ok = false; break; }
            load4(v_smem, &map_v, &map_vt, v_full, it.row0 + (it.j0 + j) * kRows);
          } else {
            const int s = t & 1;
            const uint32_t ph = (t >> 1) & 1;
            if (!mbar_wait(k_empty + 8 * s, ph ^ 1, abort_ptr)) { give_up(0x11); ok = false; break; }
            mbar_expect_tx(k_full + 8 * s, kTileBytes);
            tma_load_3d(k_smem + s * kTileBytes, &map_k, k_full + 8 * s, 0, it.row0 + (it.j0 + j) * kRows, it.h);
            if (!BF16) tma_load_3d(k_smem + s * kTileBytes + kSlab, &map_k, k_full + 8 * s, 32, it.row0 + (it.j0 + j) * kRows, it.h);
            if (!mbar_wait(v_empty + 8 * s, ph ^ 1, abort_ptr)) { give_up(0x12); ok = false; break; }
            mbar_expect_tx(v_full + 8 * s, kTileBytes);
            tma_load_3d(v_smem + s * kTileBytes, &map_v, v_full + 8 * s, 0, it.row0 + (it.j0 + j) * kRows, it.h);
            if (!BF16) tma_load_3d(v_smem + s * kTileBytes + kSlab, &map_v, v_full + 8 * s, 32, it.row0 + (it.j0 + j) * kRows, it.h);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      bool ok = true;
      // Tiles are numbered over all items (t): ring slot, S buffer and O_part buffer are t & 1, phases (t >> 1) & 1
      // (EXACT: the single K and V buffers change phase with every tile).
      auto issue_qk = [&](int t) {
        const int s = t & 1;
        if (!mbar_wait(EXACT ? k_full : k_full + 8 * s, EXACT ? (t & 1) : ((t >> 1) & 1), abort_ptr)) { give_up(0x22); ok = false; return; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t kb = EXACT ? k_smem : k_smem + s * kTileBytes;
        // 32 bytes of the head dimension per instruction: 8 float32 (TF32) or 16 bf16
        if constexpr (EXACT) {
          // heads x heads, heads x tails, tails x heads
#pragma unroll
          for (int pass = 0; pass < 3; ++pass) {
            const uint32_t qa = q_smem + (pass == 2 ? kTileBytes : 0), ka = kb + (pass == 1 ? kTileBytes : 0);
#pragma unroll
            for (int kd = 0; kd < kTileSlabs * 4; ++kd) {
              const uint32_t off = (uint32_t)(kd >> 2) * kSlab + (uint32_t)(kd & 3) * 32;
              umma(tmem_base + (uint32_t)s * 128, make_desc(qa + off, 16, 1024), make_desc(ka + off, 16, 1024), p.idesc_qk,
                   (pass | kd) != 0 ? 1u : 0u, false);
            }
          }
        } else {
#pragma unroll
          for (int kd = 0; kd < kTileSlabs * 4; ++kd) {
            const uint32_t off = (uint32_t)(kd >> 2) * kSlab + (uint32_t)(kd & 3) * 32;
            umma(tmem_base + (uint32_t)s * 128, make_desc(q_smem + off, 16, 1024), make_desc(kb + off, 16, 1024), p.idesc_qk,
                 kd != 0 ? 1u : 0u, BF16);
          }
        }
        umma_commit(sfull0 + 8 * s);
        umma_commit(EXACT ? k_empty : k_empty + 8 * s);
      };
      // P V of tile t: the 128 keys of both threads of a row pair into the O_part buffer (t & 1), as two
      // runs of MMAs (a group's P occupies the first columns of its 64-column share of S).  In-order
      // execution of the tensor pipe keeps S[s] intact until these reads of P are done (the next Q K^T
      // into S[s] is issued later), and the buffer (t & 1) was folded by the softmax threads before
      // they published P of tile t.
      auto issue_pv = [&](int t) {
        const int s = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(EXACT ? v_full : v_full + 8 * s, EXACT ? (uint32_t)(t & 1) : ph, abort_ptr)) { give_up(0x23); ok = false; return; }
        const uint32_t vb = EXACT ? v_smem : v_smem + s * kTileBytes;
        const uint32_t o_addr = tmem_o0 + (uint32_t)s * 64;
        for (int g = 0; g < 2; ++g) {
          if (!mbar_wait(pfull0 + 8 * (g * 2 + s), ph, abort_ptr)) { give_up(0x24); ok = false; return; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if constexpr (EXACT) {
            // P x V, P x tails of V, tails of P x V
#pragma unroll
            for (int pass = 0; pass < 3; ++pass) {
              const uint32_t pa = pass == 2 ? tmem_pt : tmem_base + (uint32_t)s * 128;
              const uint32_t va = vb + (pass == 1 ? kTileBytes : 0);
#pragma unroll
              for (int kk = 0; kk < 8; ++kk)
                umma_ts(o_addr, pa + (uint32_t)(g * 64 + kk * 8), make_desc(va + (uint32_t)(g * 8 + kk) * 1024, kSlab, 512, 1),
                        p.idesc_pv, (g | kk | pass) != 0 ? 1u : 0u, false);
            }
          } else if (BF16) {
            // P: two bf16 per TMEM column, 16 keys = 8 columns per instruction; V: [keys x 64 dims] bf16,
            // one 128-byte swizzled row per key, 16 rows per instruction
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
              umma_ts(o_addr, tmem_base + (uint32_t)s * 128 + (uint32_t)(g * 64 + kk * 8),
                      make_desc(vb + (uint32_t)(g * 4 + kk) * 2048, kSlab, 1024, 2), p.idesc_pv, (g | kk) != 0 ? 1u : 0u, true);
          } else {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk)
              umma_ts(o_addr, tmem_base + (uint32_t)s * 128 + (uint32_t)(g * 64 + kk * 8),
                      make_desc(vb + (uint32_t)(g * 8 + kk) * 1024, kSlab, 512, 1), p.idesc_pv, (g | kk) != 0 ? 1u : 0u, false);
          }
        }
        umma_commit(ofull0 + 8 * s);
        umma_commit(EXACT ? v_empty : v_empty + 8 * s);
      };
      // An item's first scores: its Q must have landed; once its last scores are issued, the Q tile is handed back.
      auto first_qk = [&](int ii, int t, int n_kv) {
        if (!mbar_wait(q_full, ii & 1, abort_ptr)) { give_up(0x21); ok = false; return; }
        issue_qk(t);
        if (ok && n_kv == 1) umma_commit(q_empty);
      };
      int t = 0;
      for (int ii = 0; ok; ++ii) {
        const int w = nth_item(ii);
        if (w < 0) break;
        const int n_kv = item_of(w).n_kv;
        // (The next item's first scores are NOT issued ahead of this item's last P V: the softmax warps
        // wait for that P V to finish the item, and have the merge and the stores to do before they
        // need the next scores.)
        first_qk(ii, t, n_kv);
        for (int j = 0; j < n_kv && ok; ++j) {
#ifdef KB200_TRACE
          ATTN_MMA_STAMP(tm); ++tm;
#endif
          if (j + 1 < n_kv) {
            issue_qk(t + j + 1);                     // the next scores are computed while the softmax warps work on tile j
            if (ok && j + 2 == n_kv) umma_commit(q_empty);
          }
#ifdef KB200_TRACE
          ATTN_MMA_STAMP(tm); ++tm;
#endif
          if (ok) issue_pv(t + j);
#ifdef KB200_TRACE
          ATTN_MMA_STAMP(tm); ++tm;
#endif
        }
        t += n_kv;
      }
    }
  } else {
    // ---------------- softmax / output (warps 2..9) ----------------
    // Two threads share a query row (TMEM lane): thread g of the pair takes keys g*64 .. g*64+63 of every
    // tile.  They keep ONE online-softmax state per row: each tile they exchange the maxima of their
    // halves through shared memory (a 64-thread barrier per lane quadrant), so both use the same
    // reference point, their probabilities go into one P V of 128 keys and one O_part, and thread g
    // folds, normalises and stores head dims g*32 .. g*32+31.  Per item only the two partial row sums
    // cross between them.
    const int quad = warp & 3;
    const int group = (warp - 2) >> 2;
    const int row = quad * 32 + lane;              // row of the tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const int c0 = group * 64;
    // behind the rings: [2 tile parities][2 groups][128 rows] maxima, [2 item parities][2][128] row sums,
    // then a staging slot per warp for the output rows (32 x 32 float32 + their bf16 copy)
    float* const xmax = reinterpret_cast<float*>(smem_raw + (v_smem - raw) + 2 * kTileBytes);
    float* const xsum = xmax + 4 * kRows;
    [[maybe_unused]] uint8_t* const stage = reinterpret_cast<uint8_t*>(xmax) + kExchangeBytes + (size_t)((warp - 2) * kStageBytes);   // (not EXACT)
    const int pair_barrier = 2 + quad;              // hardware barriers 2..5, 64 threads each
    // The pair's barrier also carries the abort flag (an OR over what the 64 threads read before they
    // arrived), so that both threads of a row take the same decision and neither waits for the other.
    auto pair_sync_aborted = [&]() {
      uint32_t any;
      asm volatile(
          "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %2, 0;\n\tbar.red.or.pred q, %1, 64, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
          : "=r"(any)
          : "r"(pair_barrier), "r"((uint32_t)*abort_ptr)
          : "memory");
      return any != 0;
    };
    bool ok = true;
    int t0 = 0;                                      // tiles of the items before this one
    for (int ii = 0; ok; ++ii) {
      const int w = nth_item(ii);
      if (w < 0) break;
      const Item it = item_of(w);
      const int n_kv = it.n_kv;
      float o[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = 0.0f;
      float m_run = -CUDART_INF_F, l_run = 0.0f, alpha_prev = 0.0f;
      // running output <- running output * alpha + this thread's 32 dims of the O_part of tile t
      auto fold = [&](int t, float alpha) {
        bool got = mbar_wait(ofull0 + 8 * (t & 1), (t >> 1) & 1, abort_ptr);
        if (!got) give_up(0x32);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        float v[32];
        tmem_ld32(tmem_o0 + lane_addr + (uint32_t)((t & 1) * 64 + group * 32), v);
        const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float2 r2 = ffma2(make_float2(o[i], o[i + 1]), alpha2, make_float2(v[i], v[i + 1]));
          o[i] = r2.x;
          o[i + 1] = r2.y;
        }
      };
      // Every thread of a pair passes the same barriers: a wait that ran out raises the CTA's flag and the
      // thread carries on to the next barrier, after which both see the flag and leave together.
      for (int j = 0; j < n_kv; ++j) {
        const int t = t0 + j;
        const int s = t & 1;
        const uint32_t ph = (t >> 1) & 1;
        if (!mbar_wait(sfull0 + 8 * s, ph, abort_ptr)) give_up(0x31);
        ATTN_STAMP(0, j);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t s_addr = tmem_base + lane_addr + (uint32_t)(s * 128 + c0);
        const bool diagonal = it.j0 + j == it.qt;
        float va[32], vb[32];
        tmem_ld32x2(s_addr, s_addr + 32, va, vb);       // both halves in flight, one wait
        // the scale is positive (checked when the chain was matched), so the maximum commutes with it
        float mx = -CUDART_INF_F;
        if (diagonal) {
          mx = row_max32<true>(va, mx, c0, row);
          mx = row_max32<true>(vb, mx, c0 + 32, row);
        } else {
          mx = row_max32<false>(va, mx, 0, 0);
          mx = row_max32<false>(vb, mx, 0, 0);
        }
        xmax[(s * 2 + group) * kRows + row] = mx;
        if (pair_sync_aborted()) { ok = false; break; }
        mx = fmaxf(mx, xmax[(s * 2 + (group ^ 1)) * kRows + row]);
        // the first key of every tile at or below the diagonal is visible to every row, so the maximum is finite
        const float m_new = fmaxf(m_run, mx * p.scale_log2);
        const float alpha = ex2(m_run - m_new);       // 0 while m_run = -inf
        float sum;
        if (diagonal) {
          sum = probabilities32<true>(va, p.scale_log2, m_new, c0, row);
          sum += probabilities32<true>(vb, p.scale_log2, m_new, c0 + 32, row);
        } else {
          sum = probabilities32<false>(va, p.scale_log2, m_new, 0, 0);
          sum += probabilities32<false>(vb, p.scale_log2, m_new, 0, 0);
        }
        if constexpr (EXACT) {
          // Fold the PREVIOUS tile's O_part first: that it is complete also says that its P V has read the
          // tails of P, whose single buffer is written next.
          if (j > 0) fold(t - 1, alpha_prev);
          ATTN_STAMP(3, j);
          const uint32_t pt_addr = tmem_pt + lane_addr + (uint32_t)c0;
          float ta[32];
          tmem_st32(s_addr, va);
#pragma unroll
          for (int i = 0; i < 32; ++i) ta[i] = va[i] - __uint_as_float(__float_as_uint(va[i]) & 0xFFFFE000u);
          tmem_st32(pt_addr, ta);
          tmem_st32(s_addr + 32, vb);
          float tb[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) tb[i] = vb[i] - __uint_as_float(__float_as_uint(vb[i]) & 0xFFFFE000u);
          tmem_st32(pt_addr + 32, tb);
        } else if (BF16) {
          // P rounded to bf16, two keys per 32-bit column: the thread's 64 keys take the first 32 columns of
          // its own 64-column share of the S buffer
          float packed[32];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(va[2 * i], va[2 * i + 1]);
            __nv_bfloat162 hi = __floats2bfloat162_rn(vb[2 * i], vb[2 * i + 1]);
            packed[i] = __uint_as_float(*reinterpret_cast<uint32_t*>(&lo));
            packed[16 + i] = __uint_as_float(*reinterpret_cast<uint32_t*>(&hi));
          }
          tmem_st32(s_addr, packed);
        } else {
          tmem_st32(s_addr, va);
          tmem_st32(s_addr + 32, vb);
        }
        tmem_st_wait();
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        mbar_arrive(pfull0 + 8 * (group * 2 + s));
        ATTN_STAMP(1, j);
        // fold the PREVIOUS tile's O_part while the tensor pipe works on this one
        if constexpr (!EXACT) {
          if (j > 0) fold(t - 1, alpha_prev);
          ATTN_STAMP(3, j);
        }
        alpha_prev = alpha;
        l_run = l_run * alpha + sum;
        m_run = m_new;
      }
      if (ok) fold(t0 + n_kv - 1, alpha_prev);
      t0 += n_kv;
      ATTN_STAMP(2, 3 * ii);
      // ---- the row sum is the two threads' partial sums; thread g normalises and stores dims g*32 .. g*32+31 ----
      xsum[((ii & 1) * 2 + group) * kRows + row] = l_run;
      if (pair_sync_aborted()) ok = false;
      ATTN_STAMP(2, 3 * ii + 1);
      // ---- a split item: leave this half's rows and state in the workspace; whoever arrives second merges.
      // Nobody waits for the other half.  The arrival is counted per lane quadrant (its 64 threads have a
      // barrier of their own, the one that also carries the abort flag), so no CTA-wide barrier is needed.
      bool writes = ok;
      float l_tot = ok ? l_run + xsum[((ii & 1) * 2 + (group ^ 1)) * kRows + row] : 1.0f;
      if (SPLIT && ok && it.split) {
        float* const mine = p.partial + ((size_t)it.slot * 2 + it.half) * kPartialFloats;
        const float* const other = p.partial + ((size_t)it.slot * 2 + (it.half ^ 1)) * kPartialFloats;
        float4* const mine4 = reinterpret_cast<float4*>(mine + row * kHeadDim + group * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i) __stcg(mine4 + i, make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]));
        if (group == 0) {
          __stcg(mine + kRows * kHeadDim + row, m_run);
          __stcg(mine + kRows * kHeadDim + kRows + row, l_tot);
        }
        __threadfence();
        if (pair_sync_aborted()) ok = false;          // the quadrant's 64 threads have written and fenced
        if (ok) {
          if (lane == 0 && group == 0) {
            arrived[quad] = atomicAdd(p.arrivals + it.slot * 4 + quad, 1);
            __threadfence();
          }
          if (pair_sync_aborted()) ok = false;
        }
        if (ok) {
          writes = arrived[quad] != 0;
          if (writes) {
            if (lane == 0 && group == 0) p.arrivals[it.slot * 4 + quad] = 0;      // for the next launch
            const float m2 = __ldcg(other + kRows * kHeadDim + row), l2 = __ldcg(other + kRows * kHeadDim + kRows + row);
            const float m = fmaxf(m_run, m2);
            const float a1 = ex2(m_run - m), a2 = ex2(m2 - m);
            // Products rounded one by one and then added (no fused multiply-add): symmetric in the two
            // halves, so the bits do not depend on which of them merges.
            l_tot = __fadd_rn(__fmul_rn(l_tot, a1), __fmul_rn(l2, a2));
            const float4* const other4 = reinterpret_cast<const float4*>(other + row * kHeadDim + group * 32);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 o2 = __ldcg(other4 + i);
              o[4 * i] = __fadd_rn(__fmul_rn(o[4 * i], a1), __fmul_rn(o2.x, a2));
              o[4 * i + 1] = __fadd_rn(__fmul_rn(o[4 * i + 1], a1), __fmul_rn(o2.y, a2));
              o[4 * i + 2] = __fadd_rn(__fmul_rn(o[4 * i + 2], a1), __fmul_rn(o2.z, a2));
              o[4 * i + 3] = __fadd_rn(__fmul_rn(o[4 * i + 3], a1), __fmul_rn(o2.w, a2));
            }
          }
        }
      }
      if (ok && writes) {
        const float inv = EXACT ? 1.0f / l_tot : __fdividef(1.0f, l_tot);
#pragma unroll
        for (int i = 0; i < 32; ++i) o[i] *= inv;
        if constexpr (EXACT) {
          // a lane holds 32 dims of ONE row: 128 contiguous bytes
          float* const dst = p.out + (int64_t)(it.row0 + it.q0 + row) * p.out_row_stride + it.h * kHeadDim + group * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
        } else {
          // A lane holds 32 dims of ONE row: the rows go through the warp's staging slot (128-byte rows, the
          // 16-byte unit XORed with the row against bank conflicts) and leave as bulk tensor stores.
          if (lane == 0) tma_store_wait_read();          // the slot's last stores have read it
          __syncwarp();
          stage_rows(stage, stage + 4096, o, lane, p.out16 != nullptr, true);
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            const int col = it.h * kHeadDim + group * 32, first_row = it.row0 + it.q0 + quad * 32;
            tma_store_3d(&map_out, smem_u32(stage), col, first_row, 0);
            if (p.out16 != nullptr) tma_store_3d(&map_out16, smem_u32(stage + 4096), col, first_row, 0);
            tma_store_commit();
          }
        }
      }
      ATTN_STAMP(2, 3 * ii + 2);
    }
    if (!EXACT && lane == 0) tma_store_wait_read();    // shared memory must outlive the stores that read it
  }

  // ---------------- common exit ----------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
#ifdef KB200_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long g;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
    printf("ATTN block0 globaltimer start %lld end %lld (ns) dur %lld | exit cycles %lld n_kv %d\n", marks[0], (long long)g,
           (long long)g - marks[0], clock64() - marks[1], item_of(blockIdx.x).n_kv);
    printf("softmax thread per item (tiles done, states exchanged, rows stored):");
    for (int j = 0; j < 15; ++j) printf(" %lld", trace[2][j] - marks[1]);
    printf("\n");
    printf("MMA thread (per tile: loop top, after Q K^T of the next tile, after P V):");
    for (int j = 0; j < 48; ++j) printf(" %lld", mma_trace[j] - marks[1]);
    printf("\n");
    for (int j = 0; j < item_of(blockIdx.x).n_kv && j < 16; ++j)
      printf("kv %2d  s_ready %7lld p_stored %7lld folded %7lld\n", j, trace[0][j] - marks[1], trace[1][j] - marks[1],
             trace[3][j] - marks[1]);
  }
#endif
  if (abort_flag && threadIdx.x == 0) {
    for (int s = 0; s < (EXACT ? 1 : 2); ++s)
      for (uint32_t i = 0; i < 4096u; ++i)
        if ((mbar_try_wait(k_full + 8 * s, 0) || mbar_try_wait(k_full + 8 * s, 1)) &&
            (mbar_try_wait(v_full + 8 * s, 0) || mbar_try_wait(v_full + 8 * s, 1)))
          break;
  }
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

struct Range {
  const float* lo;
  const float* hi;
};

Range out_range(const PlanKernel& k, int slot) {
  const kb200_kernel_desc& d = k.desc;
  int64_t span = 0;
  for (int i = 0; i < d.iter_rank; ++i) span += (d.iter_shape[i] - 1) * k.ops[slot].stride[i];
  return {k.ops[slot].ptr, k.ops[slot].ptr + span + 1};
}

bool overlaps(Range a, Range b) { return a.lo < b.hi && b.lo < a.hi; }
bool covers(Range a, Range b) { return a.lo <= b.lo && a.hi >= b.hi; }

// Operand slots a kernel reads / writes.
void io_slots(const PlanKernel& k, std::vector<int>* reads, std::vector<int>* writes) {
  const kb200_kernel_desc& d = k.desc;
  if (d.kclass == KB200_K_MATMUL) {
    reads->push_back(d.a_slot);
    reads->push_back(d.b_slot);
  }
  for (int t = 0; t < d.n_tape; ++t) {
    if (d.tape[t].opcode == KB200_OP_LOAD) reads->push_back(d.tape[t].a);
    if (d.tape[t].opcode == KB200_OP_STORE) writes->push_back(d.tape[t].b);
  }
  for (int slot = d.n_operands; slot < k.n_ops; ++slot) reads->push_back(slot);   // side operands of an absorbed kernel
}

Range operand_range(const PlanKernel& k, int slot) {
  const kb200_kernel_desc& d = k.desc;
  int64_t ext[KB200_MAX_RANK];
  for (int i = 0; i < d.iter_rank; ++i) ext[i] = d.iter_shape[i];
  if (d.kclass == KB200_K_MATMUL) {
    if (slot == d.a_slot) ext[2] = d.k_extent;
    if (slot == d.b_slot) { ext[1] = d.k_extent; ext[2] = d.iter_shape[2]; }
  }
  int64_t span = 0;
  for (int i = 0; i < d.iter_rank; ++i) span += (ext[i] - 1) * k.ops[slot].stride[i];
  return {k.ops[slot].ptr, k.ops[slot].ptr + span + 1};
}

bool is_copy(const PlanKernel& k) {
  return k.desc.kclass == KB200_K_ELEMENTWISE && k.has_chain && k.chain.n == 1 && k.chain.steps[0].op == CH_COPY &&
         k.chain.first_slot >= 0;
}

}  // namespace

namespace {

// What both matchers below hand to the common part.
struct AttnChain {
  size_t first = 0;
  int count = 0;                      // plan kernels covered: first .. first + count - 1
  int64_t B = 1, H = 0, T = 0, rs = 0; // sequences, heads, tokens, row stride of the Q / K / V views
  const float* q = nullptr;
  const float* k = nullptr;
  const float* v = nullptr;
  float scale = 0.f;
  const DevOperand* mask = nullptr;
  const DevOperand* y = nullptr;      // the merged-heads output, rows of H * 64
  Range y_range{nullptr, nullptr};
  std::vector<Range> dead;            // intermediates the fused kernel never writes
  std::vector<Range> sources;         // what the fused kernel reads (Q, K, V views)
  std::vector<PlanKernel*> matmuls;   // tensor-core state to drop
  bool bf16 = false;
  bool exact = false;                 // the chain's matmuls are in FP32 mode
  bool ieee = false;                  // ... and were asked to behave like FMA matmuls on non-finite operands (config bit 1024)
};

// Shared tail of the two matchers: the intermediates must be dead afterwards, the mask causal; then
// the state is built and the plan kernels are marked.
bool finish_fusion(Plan& plan, const AttnChain& c) {
  const int64_t T = c.T, H = c.H, B = c.B, hd = kHeadDim, rs = c.rs;
  if (!aligned16(c.q) || !aligned16(c.k) || !aligned16(c.v) || !aligned16(c.y->ptr)) return false;
  if (B * H * (T / kRows) >= (int64_t(1) << 31)) return false;
  // A later read that touches an intermediate is only acceptable if everything it reads was rewritten
  // after the chain (by the chain's own output Y, whose memory the planner may have taken from
  // them, or by a later kernel).
  {
    std::vector<Range> rewritten{c.y_range};
    for (size_t j = c.first + c.count; j < plan.kernels.size(); ++j) {
      std::vector<int> reads, writes;
      io_slots(plan.kernels[j], &reads, &writes);
      for (int slot : reads) {
        const Range r = operand_range(plan.kernels[j], slot);
        bool touches = false;
        for (const Range& d : c.dead) touches = touches || overlaps(r, d);
        if (!touches) continue;
        bool fresh = false;
        for (const Range& w : rewritten) fresh = fresh || covers(w, r);
        if (!fresh) return false;
      }
      for (int slot : writes) rewritten.push_back(operand_range(plan.kernels[j], slot));
    }
  }
  // the fused kernel writes Y while other CTAs still read Q, K, V: if the planner reused their
  // memory for Y, the result is staged in a private buffer and copied afterwards
  bool aliased = false;
  for (const Range& src : c.sources) aliased = aliased || overlaps(c.y_range, src);

  // --- the mask must be the causal one: 0 on and below the diagonal, -inf above ---
  {
    std::vector<float> host((size_t)T * T);
    if (cudaMemcpy(host.data(), c.mask->ptr, host.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess) {
      cudaGetLastError();
      return false;
    }
    for (int64_t r = 0; r < T; ++r)
      for (int64_t col = 0; col < T; ++col) {
        const float v = host[(size_t)r * T + col];
        if (col <= r ? v != 0.0f : !(v < 0.0f && isinf(v))) return false;
      }
  }

  // Q, K, V as [head, row, 64] views with rows b * T + t: a batch of sequences is more rows of the same map
  AttnState* st = new AttnState();
  st->exact = c.exact;
  // FP32 mode: the tensor-core kernel when its work items (128 queries each) fill at least a quarter
  // of the SMs, the CUDA-core kernel (64 queries per CTA, long prefixes split) for the short sequences
  // below that (one 128-token sequence: 8.6 against 10.4 us; 512 tokens: 22.4 against 20.9);
  // the plan option KB200_OPT_FP32_ATTENTION forces one of them.
  if (c.exact) {
    // (split operands turn an infinite element into a NaN tail: a plan that asked for IEEE behaviour keeps the FMA kernel)
    st->exact_tc = !c.ieee && B * H * (T / kRows) * 4 >= plan.sm_count;
    if (plan.fp32_attention == 1) st->exact_tc = false;
    if (plan.fp32_attention == 2) st->exact_tc = true;
  }
  if ((!c.exact || st->exact_tc) && (!encode_map(&st->map_q, false, c.q, hd, B * T, H, rs, hd, 32, kRows, false) ||
                                     !encode_map(&st->map_k, false, c.k, hd, B * T, H, rs, hd, 32, kRows, false) ||
                                     !encode_map(&st->map_v, false, c.v, hd, B * T, H, rs, hd, 32, kRows, true))) {
    delete st;
    return false;
  }
  if (st->exact_tc) {
    // the tails of everything the three views cover, in a buffer of the same shape
    const float* lo = c.q < c.k ? c.q : c.k;
    if (c.v < lo) lo = c.v;
    const float* last = c.q > c.k ? c.q : c.k;
    if (c.v > last) last = c.v;
    const int64_t span = (last - lo) + (B * T - 1) * rs + H * hd;
    st->span_lo = lo;
    st->span_n4 = span / 4;
    const bool ok = span % 4 == 0 && cudaMalloc(&st->tails, (size_t)span * sizeof(float)) == cudaSuccess &&
                    encode_map(&st->map_qt, false, st->tails + (c.q - lo), hd, B * T, H, rs, hd, 32, kRows, false) &&
                    encode_map(&st->map_kt, false, st->tails + (c.k - lo), hd, B * T, H, rs, hd, 32, kRows, false) &&
                    encode_map(&st->map_vt, false, st->tails + (c.v - lo), hd, B * T, H, rs, hd, 32, kRows, true) &&
                    cudaFuncSetAttribute(attention_kernel<false, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kExactSmemBytes) == cudaSuccess &&
                    cudaFuncSetAttribute(attention_kernel<false, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         kExactSmemBytes) == cudaSuccess;
    if (!ok) {
      cudaGetLastError();
      if (st->tails) cudaFree(st->tails);
      delete st;
      return false;
    }
  }
  if (cudaFuncSetAttribute(attention_kernel<false, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn_smem(false)) != cudaSuccess ||
      cudaFuncSetAttribute(attention_kernel<false, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn_smem(false)) != cudaSuccess ||
      cudaFuncSetAttribute(attention_fp32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFSmemBytes) != cudaSuccess ||
      cudaFuncSetAttribute(attention_kernel<true, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn_smem(true)) != cudaSuccess ||
      cudaFuncSetAttribute(attention_kernel<true, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, attn_smem(true)) != cudaSuccess) {
    cudaGetLastError();
    delete st;
    return false;
  }
  st->q_ptr = c.q;
  st->k_ptr = c.k;
  st->v_ptr = c.v;
  st->row_stride = rs;
  st->chain = c.count;
  st->wants_bf16 = c.bf16;
  AttnParams& p = st->params;
  p.T = (int)T;
  p.H = (int)H;
  p.B = (int)B;
  p.q_tiles = (int)(T / kRows);
  p.scale_log2 = c.scale * 1.4426950408889634f;
  p.out = c.y->ptr;
  p.out_row_stride = H * hd;
  p.out16 = nullptr;
  p.out16_row_stride = H * hd;
  st->y = c.y;
  st->y_elems = B * T * H * hd;
  if (aliased) {
    st->out_elems = B * T * H * hd;
    if (cudaMalloc(&st->staged_out, (size_t)st->out_elems * sizeof(float)) != cudaSuccess) {
      cudaGetLastError();
      if (st->tails) cudaFree(st->tails);
      delete st;
      return false;
    }
    st->final_out = c.y->ptr;
    p.out = st->staged_out;
  }
  // D = F32, A/B = TF32, both K-major, N = 128 | B N-major, N = 64; M = 128
  p.idesc_qk = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(kRows >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
  p.idesc_pv = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 16) | ((uint32_t)(kHeadDim >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
  p.kernel_index = (int)c.first;
  p.status = plan.d_status;
  // the output rows leave by bulk tensor stores: [B * T, H * 64], boxes of 32 rows x 32 dims
  if (!aligned16(p.out) || !encode_map_store(&st->map_out, false, p.out, H * hd, B * T, 1, p.out_row_stride, 0)) {
    if (st->staged_out) cudaFree(st->staged_out);
    if (st->tails) cudaFree(st->tails);
    delete st;
    return false;
  }
  st->map_out16 = st->map_out;
  // When the items do not fill the persistent CTAs, the launch takes as long as its longest item: the
  // upper half of the query tiles is then shared by two CTAs each (one sequence of 1024 tokens: 96
  // items of 1..8 key tiles become 144 of at most 4).  A split item costs about three BF16 key tiles
  // (partial rows out, fence, counter, the other half's rows in), so it pays only for long items in an
  // underfilled launch -- measured, one sequence: BF16 1024 tokens 14.4 -> 13.4 us but 512 tokens 9.6
  // -> 10.8 and 2048 tokens (192 items, two rounds) 24.4 -> 29.4; FP32 mode, whose tiles take three
  // times the MMAs, 1024 tokens 37.0 -> 28.1 and 2048 tokens 67.8 -> 65.4.
  p.split_from = p.q_tiles;
  p.partial = nullptr;
  p.arrivals = nullptr;
  p.order = nullptr;
  if (!(c.exact && !st->exact_tc) && p.q_tiles >= 8 && B * H * p.q_tiles <= (c.exact ? 2 : 1) * (int64_t)plan.sm_count &&
      plan.concurrency == 1 &&                       // other plans in flight fill the SMs this one leaves idle
      plan.attention_split) {
    p.split_from = p.q_tiles / 2;
    const int64_t split_tiles = B * H * (p.q_tiles - p.split_from);
    const size_t partial_bytes = (size_t)split_tiles * 2 * kPartialFloats * sizeof(float);
    const size_t counter_bytes = (size_t)split_tiles * 4 * sizeof(int);
    // whole tiles and halves by descending number of key tiles, so that the alternating rounds of the
    // persistent CTAs pair a long item with a short one
    std::vector<std::pair<int, unsigned short>> entries;
    for (int qt = 0; qt < p.q_tiles; ++qt) {
      const int n = qt + 1;
      if (qt >= p.split_from) {
        entries.push_back({n >> 1, (unsigned short)(qt << 1)});
        entries.push_back({n - (n >> 1), (unsigned short)(qt << 1 | 1)});
      } else {
        entries.push_back({n, (unsigned short)(qt << 1)});
      }
    }
    std::stable_sort(entries.begin(), entries.end(), [](const auto& a, const auto& b) { return a.first > b.first; });
    std::vector<unsigned short> order;
    for (const auto& e : entries) order.push_back(e.second);
    const size_t order_bytes = (order.size() * sizeof(unsigned short) + 15) & ~size_t(15);
    if (cudaMalloc(&st->split_scratch, partial_bytes + counter_bytes + order_bytes) != cudaSuccess ||
        cudaMemset(static_cast<uint8_t*>(st->split_scratch) + partial_bytes, 0, counter_bytes) != cudaSuccess ||
        cudaMemcpy(static_cast<uint8_t*>(st->split_scratch) + partial_bytes + counter_bytes, order.data(),
                   order.size() * sizeof(unsigned short), cudaMemcpyHostToDevice) != cudaSuccess) {
      cudaGetLastError();
      if (st->split_scratch) cudaFree(st->split_scratch);
      if (st->staged_out) cudaFree(st->staged_out);
      if (st->tails) cudaFree(st->tails);
      delete st;
      return false;
    }
    p.partial = static_cast<float*>(st->split_scratch);
    p.arrivals = reinterpret_cast<int*>(static_cast<uint8_t*>(st->split_scratch) + partial_bytes);
    p.order = reinterpret_cast<const unsigned short*>(static_cast<uint8_t*>(st->split_scratch) + partial_bytes + counter_bytes);
  }
  const int64_t items = B * H * (p.q_tiles + (p.q_tiles - p.split_from));
  st->grid = dim3((unsigned)(items < plan.sm_count ? items : plan.sm_count), 1, 1);     // persistent: at most one CTA per SM
  if (c.exact && !st->exact_tc) {
    AttnF32Params& f = st->f32;
    f.q = c.q; f.k = c.k; f.v = c.v;
    f.row_stride = rs;
    f.out = p.out;
    f.out_row_stride = p.out_row_stride;
    f.T = (int)T; f.H = (int)H; f.B = (int)B;
    f.q_tiles = (int)(T / kFTile);
    f.scale_log2 = p.scale_log2;
    // the upper half of the query tiles (the longest causal prefixes) is shared by two CTAs each
    f.split_from = f.q_tiles >= 2 ? f.q_tiles / 2 : f.q_tiles;
    const int64_t n_split = f.q_tiles - f.split_from, split_items = B * H * n_split;
    f.partial = nullptr;
    f.arrivals = nullptr;
    if (split_items > 0) {
      const size_t partial_bytes = (size_t)split_items * 2 * kFPartialFloats * sizeof(float);
      if (cudaMalloc(&st->f32_scratch, partial_bytes + (size_t)split_items * sizeof(int)) != cudaSuccess ||
          cudaMemset(static_cast<uint8_t*>(st->f32_scratch) + partial_bytes, 0, (size_t)split_items * sizeof(int)) != cudaSuccess) {
        cudaGetLastError();
        if (st->f32_scratch) cudaFree(st->f32_scratch);
        if (st->staged_out) cudaFree(st->staged_out);
        delete st;
        return false;
      }
      f.partial = static_cast<float*>(st->f32_scratch);
      f.arrivals = reinterpret_cast<int*>(static_cast<uint8_t*>(st->f32_scratch) + partial_bytes);
    }
    st->grid = dim3((unsigned)(B * H * (f.q_tiles + n_split)), 1, 1);    // a CTA per (sequence, head, 64 queries[, half of the keys])
  }

  for (PlanKernel* k : c.matmuls) destroy_matmul(*k);
  PlanKernel& holder = plan.kernels[c.first];
  holder.attn = st;
  holder.impl = IMPL_ATTN_FUSED;
  holder.launches = (aliased ? 2 : 1) + (st->exact_tc ? 1 : 0);
  for (int j = 1; j < c.count; ++j) {
    plan.kernels[c.first + j].impl = IMPL_FUSED_AWAY;
    plan.kernels[c.first + j].launches = 0;
  }
  return true;
}

// One sequence: kernels i .. i+4 (K^T copy, Q K^T * scale + mask, softmax, P V, head merge).
bool try_fuse_single(Plan& plan, size_t i) {
  if (i + 4 >= plan.kernels.size()) return false;
  PlanKernel& k2 = plan.kernels[i];
  PlanKernel& k3 = plan.kernels[i + 1];
  PlanKernel& k4 = plan.kernels[i + 2];
  PlanKernel& k5 = plan.kernels[i + 3];
  PlanKernel& k6 = plan.kernels[i + 4];
  // --- k3: scores = Q K^T * scale + mask ---
  if (k3.desc.kclass != KB200_K_MATMUL || !k3.has_chain) return false;
  const int64_t H = k3.batch, T = k3.M, hd = k3.K;
  if (hd != kHeadDim || k3.N != T || T % kRows != 0 || T < kRows || H < 1 || H > 65535) return false;
  const DevOperand& Q = k3.ops[k3.desc.a_slot];
  const DevOperand& Kt = k3.ops[k3.desc.b_slot];
  const int64_t rs = Q.stride[1];
  if (Q.stride[2] != 1 || Q.stride[0] != hd || rs % 4 || rs < H * hd) return false;
  if (Kt.stride[0] != hd * T || Kt.stride[1] != T || Kt.stride[2] != 1) return false;
  if (k3.chain.n != 2 || k3.chain.steps[0].op != CH_MUL || k3.chain.steps[0].slot != -1 || k3.chain.steps[1].op != CH_ADD ||
      k3.chain.steps[1].slot < 0)
    return false;
  const float scale = k3.chain.steps[0].imm;
  const DevOperand& mask = k3.ops[k3.chain.steps[1].slot];
  if (!(scale > 0.0f) || mask.stride[0] != 0 || mask.stride[1] != T || mask.stride[2] != 1) return false;
  if (k3.desc.operands[k3.chain.steps[1].slot].base_kind != KB200_BASE_CONST) return false;
  const DevOperand& S = k3.ops[k3.chain.out_slot];
  if (S.stride[0] != T * T || S.stride[1] != T || S.stride[2] != 1) return false;
  // --- k2: K^T = copy of the K view ---
  if (!is_copy(k2) || k2.desc.iter_rank != 2 || k2.desc.iter_shape[0] != H * hd || k2.desc.iter_shape[1] != T) return false;
  const DevOperand& Ksrc = k2.ops[k2.chain.first_slot];
  const DevOperand& Kdst = k2.ops[k2.chain.out_slot];
  if (Ksrc.stride[0] != 1 || Ksrc.stride[1] != rs || Kdst.stride[0] != T || Kdst.stride[1] != 1 || Kdst.ptr != Kt.ptr) return false;
  // --- k4: softmax over the last dim ---
  if (k4.desc.kclass != KB200_K_ROW || k4.impl != IMPL_ROW_SOFTMAX || k4.row_pre.n != 0) return false;
  if (k4.ops[k4.x_slot].ptr != S.ptr || k4.desc.iter_rank != 2 || k4.desc.iter_shape[0] != H * T || k4.desc.iter_shape[1] != T) return false;
  const DevOperand& P = k4.ops[k4.out_slot];
  if (P.stride[0] != T || P.stride[1] != 1) return false;
  // --- k5: O = P V ---
  if (k5.desc.kclass != KB200_K_MATMUL || !k5.has_chain || k5.chain.n != 0) return false;
  if ((k5.desc.precision == KB200_PREC_FP32) != (k3.desc.precision == KB200_PREC_FP32)) return false;
  if (k5.batch != H || k5.M != T || k5.N != hd || k5.K != T) return false;
  const DevOperand& Pa = k5.ops[k5.desc.a_slot];
  const DevOperand& V = k5.ops[k5.desc.b_slot];
  if (Pa.ptr != P.ptr || Pa.stride[0] != T * T || Pa.stride[1] != T || Pa.stride[2] != 1) return false;
  if (V.stride[0] != hd || V.stride[1] != rs || V.stride[2] != 1) return false;
  const DevOperand& O = k5.ops[k5.chain.out_slot];
  if (O.stride[0] != T * hd || O.stride[1] != hd || O.stride[2] != 1) return false;
  // --- k6: merge heads ---
  if (!is_copy(k6) || k6.desc.iter_rank != 3 || k6.desc.iter_shape[0] != T || k6.desc.iter_shape[1] != H ||
      k6.desc.iter_shape[2] != hd)
    return false;
  const DevOperand& Osrc = k6.ops[k6.chain.first_slot];
  const DevOperand& Y = k6.ops[k6.chain.out_slot];
  if (Osrc.ptr != O.ptr || Osrc.stride[0] != hd || Osrc.stride[1] != T * hd || Osrc.stride[2] != 1) return false;
  if (Y.stride[0] != H * hd || Y.stride[1] != hd || Y.stride[2] != 1) return false;
  // --- the four intermediates (K^T, scores, probabilities, per-head O) must be arena buffers: a graph
  // result lives in a caller's output buffer (kiln/passes/buffers.py:161,193), which the fused kernel
  // would never write ---
  if (k2.desc.operands[k2.chain.out_slot].base_kind != KB200_BASE_ARENA ||
      k3.desc.operands[k3.chain.out_slot].base_kind != KB200_BASE_ARENA ||
      k4.desc.operands[k4.out_slot].base_kind != KB200_BASE_ARENA ||
      k5.desc.operands[k5.chain.out_slot].base_kind != KB200_BASE_ARENA)
    return false;
  AttnChain c;
  c.first = i;
  c.count = 5;
  c.H = H; c.T = T; c.rs = rs;
  c.q = Q.ptr; c.k = Ksrc.ptr; c.v = V.ptr;
  c.scale = scale;
  c.mask = &mask;
  c.y = &Y;
  c.y_range = out_range(k6, k6.chain.out_slot);
  c.dead = {out_range(k2, k2.chain.out_slot), operand_range(k3, k3.chain.out_slot), out_range(k4, k4.out_slot),
            operand_range(k5, k5.chain.out_slot)};
  c.sources = {operand_range(k3, k3.desc.a_slot), operand_range(k5, k5.desc.b_slot), operand_range(k2, k2.chain.first_slot)};
  c.matmuls = {&k3, &k5};
  c.bf16 = k3.desc.precision == KB200_PREC_BF16;
  c.exact = k3.desc.precision == KB200_PREC_FP32;
  c.ieee = (k3.desc.cfg[6] & 1024) != 0;
  return finish_fusion(plan, c);
}

// A batch of sequences in one graph ([batch, tokens, d] models): kernels i .. i+6.  The buffer pass
// makes every operand of the two batched matmuls contiguous first (kiln/passes/buffers.py:208-217), and
// the fusion pass puts scale and mask in front of the softmax instead of behind the matmul:
//   i    copy  Q view   [B, H, T, 64] of the QKV projection's [B * T, 3 d] output -> contiguous
//   i+1  copy  K^T view [B, H * 64, T]                                            -> contiguous
//   i+2  matmul [B * H, T, T] = Q K^T, no epilogue
//   i+3  row    softmax(S * scale + mask)
//   i+4  copy  V view   [B, H, T, 64]                                             -> contiguous
//   i+5  matmul [B * H, T, 64] = P V
//   i+6  copy  merge heads [B, T, H, 64] -> [B * T, d]
// The fused kernel reads the three VIEWS (rows b * T + t of one [B * T, 3 d] buffer) and writes the
// merged output; none of the six intermediates is ever written.
bool try_fuse_batched(Plan& plan, size_t i) {
  if (i + 6 >= plan.kernels.size()) return false;
  PlanKernel& cq = plan.kernels[i];
  PlanKernel& ck = plan.kernels[i + 1];
  PlanKernel& mm1 = plan.kernels[i + 2];
  PlanKernel& sm = plan.kernels[i + 3];
  PlanKernel& cv = plan.kernels[i + 4];
  PlanKernel& mm2 = plan.kernels[i + 5];
  PlanKernel& merge = plan.kernels[i + 6];
  const int64_t hd = kHeadDim;
  // --- scores ---
  if (mm1.desc.kclass != KB200_K_MATMUL || !mm1.has_chain || mm1.chain.n != 0) return false;
  const int64_t BH = mm1.batch, T = mm1.M;
  if (mm1.K != hd || mm1.N != T || T % kRows != 0 || T < kRows) return false;
  const DevOperand& Qc = mm1.ops[mm1.desc.a_slot];
  const DevOperand& Ktc = mm1.ops[mm1.desc.b_slot];
  const DevOperand& S = mm1.ops[mm1.chain.out_slot];
  if (Qc.stride[0] != T * hd || Qc.stride[1] != hd || Qc.stride[2] != 1) return false;
  if (Ktc.stride[0] != hd * T || Ktc.stride[1] != T || Ktc.stride[2] != 1) return false;
  if (S.stride[0] != T * T || S.stride[1] != T || S.stride[2] != 1) return false;
  // --- the copy of Q: [B, H, T, 64] ---
  if (!is_copy(cq) || cq.desc.iter_rank != 4 || cq.desc.iter_shape[2] != T || cq.desc.iter_shape[3] != hd) return false;
  const int64_t B = cq.desc.iter_shape[0], H = cq.desc.iter_shape[1];
  if (B < 1 || H < 1 || H > 65535 || B * H != BH) return false;
  const DevOperand& Qsrc = cq.ops[cq.chain.first_slot];
  const DevOperand& Qdst = cq.ops[cq.chain.out_slot];
  const int64_t rs = Qsrc.stride[2];
  if (Qdst.ptr != Qc.ptr || Qdst.stride[0] != H * T * hd || Qdst.stride[1] != T * hd || Qdst.stride[2] != hd || Qdst.stride[3] != 1) return false;
  if (Qsrc.stride[3] != 1 || Qsrc.stride[1] != hd || rs % 4 || rs < H * hd || Qsrc.stride[0] != T * rs) return false;
  // --- the copy of K^T: [B, H * 64, T] ---
  if (!is_copy(ck) || ck.desc.iter_rank != 3 || ck.desc.iter_shape[0] != B || ck.desc.iter_shape[1] != H * hd || ck.desc.iter_shape[2] != T)
    return false;
  const DevOperand& Ksrc = ck.ops[ck.chain.first_slot];
  const DevOperand& Kdst = ck.ops[ck.chain.out_slot];
  if (Kdst.ptr != Ktc.ptr || Kdst.stride[0] != H * hd * T || Kdst.stride[1] != T || Kdst.stride[2] != 1) return false;
  if (Ksrc.stride[0] != T * rs || Ksrc.stride[1] != 1 || Ksrc.stride[2] != rs) return false;
  // --- softmax(S * scale + mask) over [B * H, T, T] ---
  if (sm.desc.kclass != KB200_K_ROW || sm.impl != IMPL_ROW_SOFTMAX || sm.desc.iter_rank != 3) return false;
  if (sm.desc.iter_shape[0] != BH || sm.desc.iter_shape[1] != T || sm.desc.iter_shape[2] != T || sm.ops[sm.x_slot].ptr != S.ptr) return false;
  if (sm.row_pre.n != 2 || sm.row_pre.steps[0].op != CH_MUL || sm.row_pre.steps[0].slot != -1 || sm.row_pre.steps[1].op != CH_ADD ||
      sm.row_pre.steps[1].slot < 0)
    return false;
  const float scale = sm.row_pre.steps[0].imm;
  const int mask_slot = sm.row_pre.steps[1].slot;
  const DevOperand& mask = sm.ops[mask_slot];
  if (!(scale > 0.0f) || mask.stride[0] != 0 || mask.stride[1] != T || mask.stride[2] != 1) return false;
  if (sm.desc.operands[mask_slot].base_kind != KB200_BASE_CONST) return false;
  const DevOperand& P = sm.ops[sm.out_slot];
  if (P.stride[0] != T * T || P.stride[1] != T || P.stride[2] != 1) return false;
  // --- the copy of V: [B, H, T, 64] ---
  if (!is_copy(cv) || cv.desc.iter_rank != 4 || cv.desc.iter_shape[0] != B || cv.desc.iter_shape[1] != H || cv.desc.iter_shape[2] != T ||
      cv.desc.iter_shape[3] != hd)
    return false;
  const DevOperand& Vsrc = cv.ops[cv.chain.first_slot];
  const DevOperand& Vdst = cv.ops[cv.chain.out_slot];
  if (Vsrc.stride[0] != T * rs || Vsrc.stride[1] != hd || Vsrc.stride[2] != rs || Vsrc.stride[3] != 1) return false;
  if (Vdst.stride[0] != H * T * hd || Vdst.stride[1] != T * hd || Vdst.stride[2] != hd || Vdst.stride[3] != 1) return false;
  // --- O = P V ---
  if (mm2.desc.kclass != KB200_K_MATMUL || !mm2.has_chain || mm2.chain.n != 0) return false;
  if ((mm2.desc.precision == KB200_PREC_FP32) != (mm1.desc.precision == KB200_PREC_FP32)) return false;
  if (mm2.batch != BH || mm2.M != T || mm2.N != hd || mm2.K != T) return false;
  const DevOperand& Pa = mm2.ops[mm2.desc.a_slot];
  const DevOperand& Vc = mm2.ops[mm2.desc.b_slot];
  const DevOperand& O = mm2.ops[mm2.chain.out_slot];
  if (Pa.ptr != P.ptr || Pa.stride[0] != T * T || Pa.stride[1] != T || Pa.stride[2] != 1) return false;
  if (Vc.ptr != Vdst.ptr || Vc.stride[0] != T * hd || Vc.stride[1] != hd || Vc.stride[2] != 1) return false;
  if (O.stride[0] != T * hd || O.stride[1] != hd || O.stride[2] != 1) return false;
  // --- merge heads: [B, T, H, 64] ---
  if (!is_copy(merge) || merge.desc.iter_rank != 4 || merge.desc.iter_shape[0] != B || merge.desc.iter_shape[1] != T ||
      merge.desc.iter_shape[2] != H || merge.desc.iter_shape[3] != hd)
    return false;
  const DevOperand& Osrc = merge.ops[merge.chain.first_slot];
  const DevOperand& Y = merge.ops[merge.chain.out_slot];
  if (Osrc.ptr != O.ptr || Osrc.stride[0] != H * T * hd || Osrc.stride[1] != hd || Osrc.stride[2] != T * hd || Osrc.stride[3] != 1) return false;
  if (Y.stride[0] != T * H * hd || Y.stride[1] != H * hd || Y.stride[2] != hd || Y.stride[3] != 1) return false;
  // --- the six intermediates must be arena buffers ---
  for (const auto& [k, slot] : {std::pair<const PlanKernel*, int>{&cq, cq.chain.out_slot}, {&ck, ck.chain.out_slot},
                                {&mm1, mm1.chain.out_slot}, {&sm, sm.out_slot}, {&cv, cv.chain.out_slot}, {&mm2, mm2.chain.out_slot}})
    if (k->desc.operands[slot].base_kind != KB200_BASE_ARENA) return false;
  AttnChain c;
  c.first = i;
  c.count = 7;
  c.B = B; c.H = H; c.T = T; c.rs = rs;
  c.q = Qsrc.ptr; c.k = Ksrc.ptr; c.v = Vsrc.ptr;
  c.scale = scale;
  c.mask = &mask;
  c.y = &Y;
  c.y_range = out_range(merge, merge.chain.out_slot);
  c.dead = {out_range(cq, cq.chain.out_slot), out_range(ck, ck.chain.out_slot), operand_range(mm1, mm1.chain.out_slot),
            out_range(sm, sm.out_slot), out_range(cv, cv.chain.out_slot), operand_range(mm2, mm2.chain.out_slot)};
  c.sources = {out_range(cq, cq.chain.first_slot), out_range(ck, ck.chain.first_slot), out_range(cv, cv.chain.first_slot)};
  c.matmuls = {&mm1, &mm2};
  c.bf16 = mm1.desc.precision == KB200_PREC_BF16;
  c.exact = mm1.desc.precision == KB200_PREC_FP32;
  c.ieee = (mm1.desc.cfg[6] & 1024) != 0;
  return finish_fusion(plan, c);
}

}  // namespace

// Tries to replace the attention chain that starts at kernel i by the fused kernel.  Returns the
// number of plan kernels it replaced (5: one sequence, 7: a batch of sequences), or 0.
int attention_try_fuse(Plan& plan, size_t i) {
  if (try_fuse_single(plan, i)) return 5;
  if (try_fuse_batched(plan, i)) return 7;
  return 0;
}

// Plan kernels the fused launch held by `k` stands for (0 if it holds none).
int attention_chain_length(const PlanKernel& k) { return k.attn ? static_cast<const AttnState*>(k.attn)->chain : 0; }
bool attention_wants_bf16(const PlanKernel& k) { return k.attn && static_cast<const AttnState*>(k.attn)->wants_bf16; }

int attention_launch(const Plan& plan, const PlanKernel& k, cudaStream_t s) {
  const AttnState* st = static_cast<const AttnState*>(k.attn);
  const bool split = st->params.split_from < st->params.q_tiles;     // some query tiles are shared by two CTAs
  if (st->exact_tc) {
    const int64_t blocks = (st->span_n4 + 255) / 256;
    KB200_CUDA(launch_kernel(plan.pdl, tails_kernel, dim3((unsigned)(blocks < 1184 ? blocks : 1184)), dim3(256), 0, s,
                             reinterpret_cast<const float4*>(st->span_lo), reinterpret_cast<float4*>(st->tails), st->span_n4));
    // (the store maps are not used by this instantiation)
    if (split)
      KB200_CUDA(launch_kernel(plan.pdl, attention_kernel<false, true, true>, st->grid, dim3(kAttnThreads), kExactSmemBytes, s, st->map_q,
                               st->map_k, st->map_v, st->map_out, st->map_out16, st->map_qt, st->map_kt, st->map_vt, st->params));
    else
      KB200_CUDA(launch_kernel(plan.pdl, attention_kernel<false, false, true>, st->grid, dim3(kAttnThreads), kExactSmemBytes, s, st->map_q,
                               st->map_k, st->map_v, st->map_out, st->map_out16, st->map_qt, st->map_kt, st->map_vt, st->params));
  } else if (st->exact) {
    KB200_CUDA(launch_kernel(plan.pdl, attention_fp32_kernel, st->grid, dim3(kFThreads), kFSmemBytes, s, st->f32));
  } else if (st->bf16) {
    // (the maps of the tails are not used by these instantiations: any valid map will do)
    if (split)
      KB200_CUDA(launch_kernel(plan.pdl, attention_kernel<true, true, false>, st->grid, dim3(kAttnThreads), attn_smem(true), s, st->map_q,
                               st->map_k, st->map_v, st->map_out, st->map_out16, st->map_q, st->map_k, st->map_v, st->params));
    else
      KB200_CUDA(launch_kernel(plan.pdl, attention_kernel<true, false, false>, st->grid, dim3(kAttnThreads), attn_smem(true), s, st->map_q,
                               st->map_k, st->map_v, st->map_out, st->map_out16, st->map_q, st->map_k, st->map_v, st->params));
  } else {
    if (split)
      KB200_CUDA(launch_kernel(plan.pdl, attention_kernel<false, true, false>, st->grid, dim3(kAttnThreads), attn_smem(false), s, st->map_q,
                               st->map_k, st->map_v, st->map_out, st->map_out16, st->map_q, st->map_k, st->map_v, st->params));
    else
      KB200_CUDA(launch_kernel(plan.pdl, attention_kernel<false, false, false>, st->grid, dim3(kAttnThreads), attn_smem(false), s, st->map_q,
                               st->map_k, st->map_v, st->map_out, st->map_out16, st->map_q, st->map_k, st->map_v, st->params));
  }
  if (st->staged_out && st->final_out) {
    const int64_t n4 = st->out_elems / 4;
    const int64_t blocks = (n4 + 255) / 256;
    KB200_CUDA(launch_kernel(plan.pdl, copy_rows_kernel, dim3((unsigned)(blocks < 1184 ? blocks : 1184)), dim3(256), 0, s,
                             reinterpret_cast<const float4*>(st->staged_out), reinterpret_cast<float4*>(st->final_out), n4));
  }
  KB200_CUDA(cudaGetLastError());
  return KB200_OK;
}

// The span of the QKV projection's output the fused kernel reads (Q, K and V are views of it).
bool attention_operand_span(const PlanKernel& k, const float** lo, const float** hi) {
  const AttnState* st = static_cast<const AttnState*>(k.attn);
  if (!st) return false;
  const float* first = st->q_ptr < st->k_ptr ? st->q_ptr : st->k_ptr;
  if (st->v_ptr < first) first = st->v_ptr;
  const float* last = st->q_ptr > st->k_ptr ? st->q_ptr : st->k_ptr;
  if (st->v_ptr > last) last = st->v_ptr;
  *lo = first;
  *hi = last + ((int64_t)st->params.B * st->params.T - 1) * st->row_stride + (int64_t)st->params.H * kHeadDim;
  return true;
}

// BF16 mode: the producer of Q, K and V also writes them as bf16 into the mirror at `mirror_base +
// (ptr - arena_base)`; read them from there (half the bytes, twice the tensor rate, P rounded to bf16).
bool attention_use_mirror(PlanKernel& k, const float* arena_base, const void* mirror_base) {
  AttnState* st = static_cast<AttnState*>(k.attn);
  if (!st) return false;
  // When the planner put the output over the QKV buffer, the output's mirror lies over the operands'
  // mirror as well: CTAs would overwrite bf16 operands others still read.  Keep the float32 operands then.
  if (st->staged_out != nullptr || st->exact) return false;
  const __nv_bfloat16* m = static_cast<const __nv_bfloat16*>(mirror_base);
  const __nv_bfloat16* q = m + (st->q_ptr - arena_base);
  const __nv_bfloat16* kk = m + (st->k_ptr - arena_base);
  const __nv_bfloat16* v = m + (st->v_ptr - arena_base);
  const int64_t T = (int64_t)st->params.B * st->params.T, H = st->params.H, rs = st->row_stride;   // rows of all sequences
  if (!aligned16(q) || !aligned16(kk) || !aligned16(v) || rs % 8) return false;
  CUtensorMap mq, mk, mv;
  if (!encode_map(&mq, true, q, kHeadDim, T, H, rs, kHeadDim, 64, kRows, false) ||
      !encode_map(&mk, true, kk, kHeadDim, T, H, rs, kHeadDim, 64, kRows, false) ||
      !encode_map(&mv, true, v, kHeadDim, T, H, rs, kHeadDim, 64, kRows, false))
    return false;
  st->map_q = mq;
  st->map_k = mk;
  st->map_v = mv;
  st->bf16 = true;
  // D = F32, A/B = BF16: Q K^T both K-major, N = 128; P V with B N-major, N = 64; M = 128
  st->params.idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kRows >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
  st->params.idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(kHeadDim >> 3) << 17) | ((uint32_t)(kRows >> 4) << 24);
  return true;
}

// When the output was staged (the planner put it over the QKV buffer), the copy back into the arena
// is only needed if someone reads the float32 output there.  Later readers that take the bf16 mirror
// do not; a tensor-core matmul whose A operand is exactly the output can read the staging buffer
// instead.  If that accounts for every reader until the buffer is rewritten (or the plan ends: arena
// contents are dead then), the copy launch is dropped.  Runs after the mirrors are assigned and
// before the matmuls build their tensor maps.
void attention_elide_copy(Plan& plan, size_t first) {
  PlanKernel& holder = plan.kernels[first];
  AttnState* st = static_cast<AttnState*>(holder.attn);
  if (!st || !st->staged_out || !st->final_out || first + st->chain - 1 >= plan.kernels.size()) return;
  const PlanKernel& k6 = plan.kernels[first + st->chain - 1];      // the head merge, whose output the fused kernel writes
  if (k6.desc.operands[k6.chain.out_slot].base_kind != KB200_BASE_ARENA) return;     // a plan output must land where the caller looks
  const int64_t width = (int64_t)st->params.H * kHeadDim;
  if (st->y->stride[st->chain == 7 ? 1 : 0] != width) return;
  const Range y{st->final_out, st->final_out + st->out_elems};
  std::vector<std::pair<PlanKernel*, int>> redirect;
  bool rewritten = false;
  for (size_t j = first + st->chain; j < plan.kernels.size() && !rewritten; ++j) {
    PlanKernel& k = plan.kernels[j];
    if (k.impl == IMPL_FUSED_AWAY) continue;
    std::vector<int> reads, writes;
    io_slots(k, &reads, &writes);
    for (int slot : reads) {
      const Range r = operand_range(k, slot);
      if (!overlaps(r, y)) continue;
      const bool is_a = k.desc.kclass == KB200_K_MATMUL && slot == k.desc.a_slot;
      const bool is_b = k.desc.kclass == KB200_K_MATMUL && slot == k.desc.b_slot;
      if (k.impl == IMPL_MM_TC && ((is_a && k.a_shadow) || (is_b && k.b_shadow))) continue;      // reads the mirror
      if (k.impl == IMPL_MM_TC && is_a && k.batch == 1 && r.lo == y.lo && r.hi == y.hi && k.ops[slot].stride[1] == width &&
          k.ops[slot].stride[2] == 1) {
        redirect.push_back({&k, slot});
        continue;
      }
      return;          // someone needs the float32 output where the plan put it
    }
    for (int slot : writes) {
      const Range w = operand_range(k, slot);
      if (covers(w, y)) rewritten = true;
      else if (overlaps(w, y)) return;                 // partly rewritten: keep it simple, keep the copy
    }
  }
  for (auto& [k, slot] : redirect) k->ops[slot].ptr = st->staged_out;
  st->final_out = nullptr;
  holder.launches = 1 + (st->exact_tc ? 1 : 0);
}

bool attention_reads_mirror(const PlanKernel& k) { return k.attn && static_cast<const AttnState*>(k.attn)->bf16; }

void attention_set_shadow(PlanKernel& k, void* shadow_out) {
  AttnState* st = static_cast<AttnState*>(k.attn);
  if (!st || st->exact) return;
  // the bf16 copy of the merged heads needs a store map of its own; without one it is not written
  // (its reader was told to expect it: assign_shadows asks attention_can_shadow first)
  __nv_bfloat16* out16 = static_cast<__nv_bfloat16*>(shadow_out);
  if (out16 != nullptr && encode_map_store(&st->map_out16, true, out16, (int64_t)st->params.H * kHeadDim,
                                            (int64_t)st->params.B * st->params.T, 1, st->params.out16_row_stride, 0))
    st->params.out16 = out16;
}

const DevOperand* attention_output(const Plan& plan, size_t first, int64_t* elems) {
  const AttnState* st = static_cast<const AttnState*>(plan.kernels[first].attn);
  *elems = st->y_elems;
  return st->y;
}

void attention_reset_arrivals(PlanKernel& k) {
  AttnState* st = static_cast<AttnState*>(k.attn);
  if (!st || !st->params.arrivals) return;
  const int64_t split_tiles = (int64_t)st->params.B * st->params.H * (st->params.q_tiles - st->params.split_from);
  cudaMemset(st->params.arrivals, 0, (size_t)split_tiles * 4 * sizeof(int));
}

void attention_destroy(PlanKernel& k) {
  if (k.attn) {
    AttnState* st = static_cast<AttnState*>(k.attn);
    if (st->staged_out) cudaFree(st->staged_out);
    if (st->f32_scratch) cudaFree(st->f32_scratch);
    if (st->tails) cudaFree(st->tails);
    if (st->split_scratch) cudaFree(st->split_scratch);
    delete st;
  }
  k.attn = nullptr;
}

}  // namespace kb200
