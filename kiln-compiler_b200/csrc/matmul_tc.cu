// Tensor-core batched matmul with fused epilogue for sm_100a: TMA -> shared-memory ring ->
// tcgen05.mma -> TMEM accumulator -> epilogue from TMEM.  Role of the reference's matmul generator
// with input_precision="tf32" (kiln/gpu/codegen.py:484-530), plus a BF16-operand mode.
//
// Persistent CTAs (one per SM) walk the list of 128 x BN output tiles; 384 threads in three roles:
//   warps 0, 10  TMA producers, one thread per operand: per pipeline stage (one or two K slabs of 128
//               bytes) boxes of A (128 rows x 128 bytes, K-major) and of B (N-major -- the layout the
//               buffer-assignment pass guarantees for B, kiln/passes/buffers.py:208-217, so nothing is
//               repacked -- or K-major), written with the 128-byte swizzle the MMA descriptors expect.
//               Plain per-CTA loads.
//   warps 1, 11  MMA issuers: one elected lane issues tcgen05.mma (M = 128, N = BN, K = 32 bytes per
//               instruction) on a stage and commits it back to the producers.  Tiles up to 128
//               columns use both, on alternate stages, each with an accumulator of its own.
//   warps 2..9  epilogue: tcgen05.ld 32 columns at a time, the fused chain on registers (bias, GELU,
//               residual, scale + mask ...), 32 x 32 blocks staged in shared memory and written with
//               bulk tensor stores.  The accumulators are double-buffered in TMEM: the epilogue of
//               tile i overlaps the main loop of tile i+1.
// A is read K-major and B N-major straight from the planned buffers (float32, consumed as TF32).
// In BF16 mode the operands are bf16: read from the mirror their producers write, or converted
// (constants once at bind, unmirrored activations per launch), and the same kernel runs with kind::f16.
// In exact-FP32 mode (allow_tf32=False: input_precision="ieee", kiln/gpu/codegen.py:515) the
// epilogue warps split every landed stage into TF32 heads and tails in shared memory, the issuer
// runs tail x head, head x tail and head x head, and a tile's K steps rotate over several TMEM
// accumulators which the epilogue adds in float32 (the tensor core truncates every accumulation).
//
// Every wait on an mbarrier is bounded.  When one runs out the thread records the site in the
// plan's status word, raises a CTA-wide abort flag, and every role falls through to the common
// exit, which waits (bounded) for copies in flight, frees the TMEM allocation and returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdio>
#include <mutex>

#include "device_math.cuh"
#include "kb200_internal.h"
#include "matmul.h"
#include "matmul_pair.h"
#include "tc_common.cuh"
#include "tc_epilogue.cuh"

namespace kb200 {

namespace {

using namespace tc;

// Experiments that change results exist in trace builds only; a shipped library ignores the bits.
#ifdef KB200_TRACE
#define KB200_EXPERIMENT(bit) (p.debug & (bit))
#else
#define KB200_EXPERIMENT(bit) false
#endif


constexpr int kTileM = 128;
constexpr int kSlabBytes = 128;           // bytes of K (A) or N (B) per swizzled row
constexpr int kATileBytes = kTileM * kSlabBytes;
constexpr int kMaxStages = 8;
constexpr int kEpiWarps = 8;
constexpr int kProducerBWarp = 2 + kEpiWarps;      // the last warp fetches operand B
constexpr int kIssuerBWarp = kProducerBWarp + 1;   // second MMA issuer (narrow tiles only)
constexpr int kThreads = 64 + 32 * kEpiWarps + 64; // producer (A) warp, MMA warp, epilogue warps, producer (B) warp, second MMA warp
// per epilogue warp: a 32 x 33 float transpose buffer, reused (as dense 32 x 32) as the staging block of
// the bulk store, then a 32 x 32 bf16 staging block; both 128-byte aligned
constexpr int kEpiStage16Offset = 4608;        // 512-byte aligned (64-byte swizzle); the float block is 1024-byte aligned
constexpr int kEpiWarpBytes = 7168;
constexpr int kEpiBytes = kEpiWarps * kEpiWarpBytes;
constexpr int kEpiSlotBytes = 4096 + 2048;   // one float block + one bf16 block of the rotating staging slots
#ifdef KB200_TRACE
constexpr int kMaxDynamicSmem = 200 * 1024;   // the trace arrays take static shared memory
#else
constexpr int kMaxDynamicSmem = 225 * 1024;   // opt-in ceiling, the same for every launch of the kernel
#endif

struct TcParams {
  // scalars the producer and MMA threads need first come first: the parameter block is read through
  // the constant cache, and every new line is a miss on the kernel's critical start-up path
  int bn;               // tile width, multiple of 32 (tf32) / 64 (bf16), <= 256
  int stages;
  int num_kb;           // K slabs
  int slab_k;           // elements of K per slab (128 bytes): 32 (tf32) or 64 (bf16)
  int kps;              // K slabs per pipeline stage (1 or 2): narrow tiles are bound by the issue cost of a stage, not its size
  int step_k;           // elements of K per stage: kps * slab_k
  int chunk_n;          // elements of N per B box: 32 (tf32) or 64 (bf16)
  int b_step_bytes;     // bytes between consecutive MMA K steps inside a B chunk
  int b_sbo_bytes;      // bytes between the row groups of one swizzle atom of B
  int b_layout;         // descriptor layout type of B (1 = 128-byte swizzle on 32-byte atoms, 2 = 128-byte swizzle)
  int b_kmajor;         // B is read K-major ([N, K] with K contiguous) like A
  int b_mode;           // how B is fetched: 0 K-major (one box), 1 N-major, all chunks in one 4-D box, 2 N-major, a box per chunk
  int debug;            // trace builds only: 1 = no stores, 16 = no epilogue (results are then wrong), 32 = no warm-up pass
  int tmem_cols;        // power of two >= bn, >= 32
  int nacc;             // exact-FP32 mode: accumulators a tile's K steps rotate over (1 otherwise)
  int acc2;             // exact-FP32 mode: the accumulators of a tile fit twice (256 columns each): two buffers
  uint32_t idesc;
  int kernel_index;
  int* status;
  int tiles_m, tiles_n, num_tiles;   // tiles per batch entry along M and N; total over the batch
  int pre_col_step, pre_mat_step;    // chain steps whose operand the epilogue fetches ahead (-1 = none)
  __nv_bfloat16* out16;              // optional bf16 copy of the output (same strides as the output), or null
  int splits;           // split-K factor: a tile's K range is shared by the CTAs of one cluster of this size
  int recv_offset;      // split K: byte offset (from the aligned tile area) of the area the neighbours push their partial bands into
  int num_units;        // num_tiles * splits
  int store_mode;       // 0: the epilogue warps store with ordinary global stores; 1: bulk tensor stores from shared memory
  int split3;           // exact-FP32 mode: every operand is split in shared memory into a TF32 head and a TF32 tail,
                        // and three MMAs per K step (head x head, head x tail, tail x head) give float32 products
  int issuers;          // 1, or 2: two threads issue the MMAs of alternate pipeline stages into accumulators of their own
  uint64_t magic_stages;   // ceil(2^40 / stages)
  int epi_rowwise;      // the epilogue keeps a lane per ROW (no transpose): the chain has no matrix operand
  int n_chunks;         // bn / chunk_n
  int tiles_per_batch;  // tiles_m * tiles_n
  uint64_t magic_tn, magic_tpb;   // ceil(2^40 / tiles_n), ceil(2^40 / tiles_per_batch): division by multiplication
  MatmulParams mm;      // shapes, operands, the epilogue chain (epilogue warps only)
};

// x / d for x, d < 2^20 with magic = ceil(2^40 / d): a lone thread pays ~100 cycles for a real division.
__device__ __forceinline__ int fast_div(int x, uint64_t magic) { return (int)(((uint64_t)(uint32_t)x * magic) >> 40); }

// Work unit -> (K split, batch entry, tile row, tile column).
__device__ __forceinline__ void unit_coords(const TcParams& p, int unit, int& tile, int& ks, int& batch, int& tm, int& tn) {
  tile = unit;
  ks = 0;
  if (p.splits > 1) {
    tile = unit / p.splits;
    ks = unit - tile * p.splits;
  }
  batch = fast_div(tile, p.magic_tpb);
  const int rem = tile - batch * p.tiles_per_batch;
  tm = fast_div(rem, p.magic_tn);
  tn = rem - tm * p.tiles_n;
}
// K slabs [begin, end) of split `ks`.
__device__ __forceinline__ void slab_range(const TcParams& p, int ks, int& begin, int& end) {
  begin = 0;
  end = p.num_kb;
  if (p.splits > 1) {
    begin = ks * p.num_kb / p.splits;
    end = (ks + 1) * p.num_kb / p.splits;
  }
}

// a = head + tail, head the 19 leading bits of a.  The tensor core reads only those bits of a TF32
// operand, so the landed float serves as its own head and only the tail (exact in float32, of which the
// tensor core again keeps the leading 11 significant bits) has to be written.
__device__ __forceinline__ float tf32_tail(float a) {
  return a - __uint_as_float(__float_as_uint(a) & 0xFFFFE000u);
}



// The epilogue works on 32 x 32 blocks of the tile after a transpose through shared memory, so
// that a lane owns one COLUMN (x[r] = row r): every global load / store of a warp then covers 128
// contiguous bytes of one row, and the 32 rows give 32 independent accesses in flight per lane.

// Side operand of chain step `s` for the block (zeros outside the matrix).
__device__ __forceinline__ void load_side32(const TcParams& p, int s, float (&side)[32], int64_t b, int64_t m_first, int64_t n,
                                            int row_limit) {
  const MatmulParams& mm = p.mm;
  const DevOperand& o = mm.ops[mm.chain.steps[s].slot];
  const bool col_ok = n < mm.N;
  int64_t rows_left = mm.M - m_first;         // may be <= 0 for a tile hanging over the bottom edge
  if (rows_left > row_limit) rows_left = row_limit;
  const float* base = o.ptr + b * o.stride[0] + m_first * o.stride[1] + n * o.stride[2];
  if (o.stride[1] == 0) {                      // one value per column (bias): a single load
    const float t = (col_ok && rows_left > 0) ? __ldg(base) : 0.0f;
#pragma unroll
    for (int r = 0; r < 32; ++r) side[r] = t;
  } else {
    const int64_t sm = o.stride[1];
#pragma unroll
    for (int r = 0; r < 32; ++r) side[r] = (col_ok && r < rows_left) ? __ldg(base + r * sm) : 0.0f;
  }
}

// Two operands of the chain are fetched ahead of the accumulator (their L2 latency then overlaps
// the main loop, the TMEM load and the previous block's stores): the first per-column operand
// (a bias: one value per lane) and the first full-matrix operand (a residual or a mask).
__device__ __forceinline__ void prefetch_col(const TcParams& p, float& pre_col, int64_t b, int64_t n) {
  const MatmulParams& mm = p.mm;
  if (p.pre_col_step >= 0) {
    const DevOperand& o = mm.ops[mm.chain.steps[p.pre_col_step].slot];
    pre_col = (n < mm.N) ? __ldg(o.ptr + b * o.stride[0] + n * o.stride[2]) : 0.0f;
  }
}
__device__ __forceinline__ void prefetch_mat(const TcParams& p, float (&pre_mat)[32], int64_t b, int64_t m_first, int64_t n,
                                             int row_limit = 32) {
  if (p.pre_mat_step >= 0) load_side32(p, p.pre_mat_step, pre_mat, b, m_first, n, row_limit);
}
__device__ __forceinline__ void prefetch_sides(const TcParams& p, float& pre_col, float (&pre_mat)[32], int64_t b,
                                               int64_t m_first, int64_t n, int row_limit = 32) {
  prefetch_col(p, pre_col, b, n);
  prefetch_mat(p, pre_mat, b, m_first, n, row_limit);
}

__device__ __forceinline__ void epilogue_compute32(const TcParams& p, float (&x)[32], float pre_col, const float (&pre_mat)[32],
                                                   int64_t b, int64_t m_first, int64_t n, int row_limit = 32) {
  const MatmulParams& mm = p.mm;
  for (int s = 0; s < mm.chain.n; ++s) {
    const ChainStep st = mm.chain.steps[s];
    if (s == p.pre_mat_step) {
      chain_step32(st.op, x, pre_mat);
    } else {
      float side[32];
      if (s == p.pre_col_step) {
#pragma unroll
        for (int r = 0; r < 32; ++r) side[r] = pre_col;
      } else if (st.slot >= 0) {
        load_side32(p, s, side, b, m_first, n, row_limit);
      } else {
#pragma unroll
        for (int r = 0; r < 32; ++r) side[r] = st.imm;
      }
      chain_step32(st.op, x, side);
    }
  }
}

__device__ __forceinline__ void epilogue_store32(const TcParams& p, const float (&x)[32], int64_t b, int64_t m_first, int64_t n,
                                                 int row_limit = 32) {
  if (KB200_EXPERIMENT(1)) return;
  const MatmulParams& mm = p.mm;
  const DevOperand& o = mm.ops[mm.chain.out_slot];
  float* out = o.ptr + b * o.stride[0] + m_first * o.stride[1] + n * o.stride[2];
  const int64_t sm = o.stride[1];
  int64_t rows_left = mm.M - m_first;
  if (rows_left > row_limit) rows_left = row_limit;
  if (n < mm.N) {
#pragma unroll
    for (int r = 0; r < 32; ++r)
      if (r < rows_left) out[r * sm] = x[r];
    if (p.out16 != nullptr) {
      __nv_bfloat16* out16 = p.out16 + b * o.stride[0] + m_first * o.stride[1] + n * o.stride[2];
#pragma unroll
      for (int r = 0; r < 32; ++r)
        if (r < rows_left) out16[r * sm] = __float2bfloat16_rn(x[r]);
    }
  }
}

#ifdef KB200_TRACE
#define KB200_STAMP(role, idx) do { if (blockIdx.x == 0 && (idx) < 160) trace[role][idx] = clock64(); } while (0)
#else
#define KB200_STAMP(role, idx) do { } while (0)
#endif

// The chain on a block held a lane per ROW (v[j] = column n + j of this lane's row): every operand is
// an immediate or one value per column, read as eight 128-bit loads from an address all lanes share.
__device__ __forceinline__ void epilogue_compute_rows(const TcParams& p, float (&v)[32], int64_t b, int64_t n) {
  const MatmulParams& mm = p.mm;
  for (int s = 0; s < mm.chain.n; ++s) {
    const ChainStep st = mm.chain.steps[s];
    float side[32];
    if (st.slot >= 0) {
      const DevOperand& o = mm.ops[st.slot];
      const float4* base = reinterpret_cast<const float4*>(o.ptr + b * o.stride[0] + n);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const float4 t = n + 4 * q < mm.N ? __ldg(base + q) : make_float4(0.f, 0.f, 0.f, 0.f);
        side[4 * q] = t.x; side[4 * q + 1] = t.y; side[4 * q + 2] = t.z; side[4 * q + 3] = t.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) side[j] = st.imm;
    }
    chain_step32(st.op, v, side);
  }
}

// Staging of a 32 x 32 block for the bulk stores, in the swizzled layouts of the store maps: float
// rows of 128 bytes with the 16-byte unit index XORed by (row & 7), bf16 rows of 64 bytes with the
// unit index XORed by ((row >> 1) & 3).  Lane = column (x[r] = row r) ...
__device__ __forceinline__ void stage_columns(uint8_t* sf, uint8_t* sh, const float (&x)[32], int lane, bool with16) {
#pragma unroll
  for (int r = 0; r < 32; ++r)
    *reinterpret_cast<float*>(sf + r * 128 + ((((lane >> 2) ^ (r & 7)) << 4) | ((lane & 3) << 2))) = x[r];
  if (with16) {
#pragma unroll
    for (int r = 0; r < 32; ++r)
      *reinterpret_cast<__nv_bfloat16*>(sh + r * 64 + ((((lane >> 3) ^ ((r >> 1) & 3)) << 4) | ((lane & 7) << 1))) =
          __float2bfloat16_rn(x[r]);
  }
}

template <bool BF16, bool SPLIT3>
__global__ void __launch_bounds__(kThreads, 1)
mm_tc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
             const __grid_constant__ CUtensorMap tma_out, const __grid_constant__ CUtensorMap tma_out16,
             const __grid_constant__ TcParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[3 * kMaxStages + 6];   // + two cluster hand-shake barriers (split K) + per-stage "operands split" barriers
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
#ifdef KB200_TRACE
  __shared__ long long trace[6][160];
  __shared__ long long marks[8];
  int tp = 0, tm = 0, te = 0;
  if (blockIdx.x <= 1 && threadIdx.x == 0) {
    unsigned long long g;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
    marks[0] = (long long)g;
    marks[1] = clock64();
  }
#endif

  // 1024-byte aligned tile area (the 128-byte swizzle pattern repeats every 1024 bytes)
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const int b_tile_bytes = p.kps * p.bn * kSlabBytes;      // B part of one stage (kps K slabs)
  const int a_stage_bytes = p.kps * kATileBytes;           // A part of one stage
  const int raw_bytes = a_stage_bytes + b_tile_bytes;       // what TMA delivers per stage
  const int stage_bytes = SPLIT3 ? 2 * raw_bytes : raw_bytes;   // exact-FP32 mode: the tails of both operands follow
  uint8_t* epi_buf = smem_raw + (tiles - raw) + (size_t)p.stages * stage_bytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[kMaxStages]);
  const uint32_t tfull0 = smem_u32(&bars[2 * kMaxStages]), tempty0 = smem_u32(&bars[2 * kMaxStages + 2]);
  const uint32_t split0 = smem_u32(&bars[2 * kMaxStages + 6]);

  if (threadIdx.x == 32) {
    // descriptor fetches overlap the set-up below instead of delaying the first copy
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
    if (p.store_mode == 1) {
      prefetch_tensormap(&tma_out);
      if (p.out16 != nullptr) prefetch_tensormap(&tma_out16);
    }
  }
  if (warp == 0) {
    // one barrier per lane: full[0..7] | empty[0..7] | tfull[0..1] | tempty[0..1]
    if (lane == 0) abort_flag = 0;
    if (lane < 2 * kMaxStages + 4)
      mbar_init(full0 + 8 * lane, lane >= 2 * kMaxStages + 2 ? kEpiWarps : (lane < kMaxStages ? 2 : (lane >= 2 * kMaxStages ? (uint32_t)p.issuers : 1)));
    else if (lane < 2 * kMaxStages + 6) mbar_init(full0 + 8 * lane, 1);   // split K: `received`, completed by the bytes the neighbours push
    if (lane < kMaxStages) mbar_init(full0 + 8 * (2 * kMaxStages + 6 + lane), kEpiWarps);  // split done: one arrival per epilogue warp
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The parameter block is read through the constant cache, cold at kernel start: touch the lines the
  // producers and the MMA thread need now, under the set-up, instead of in front of the first copy.
  if (lane == 0 && (warp <= 1 || warp >= kProducerBWarp))
    asm volatile("" ::"r"(p.bn), "r"(p.tmem_cols), "r"(p.idesc), "r"(p.num_tiles), "l"(p.magic_stages), "l"(p.magic_tn), "l"(p.magic_tpb)
                 : "memory");
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
  // Split K: the hand-shake barriers of every CTA of the cluster must exist before a neighbour arrives
  // on them.  Arrive on the hardware cluster barrier now, wait for it only when the main loop is over
  // (the barrier itself takes thousands of cycles to complete; they pass under the main loop).
  if (p.splits > 1) cluster_arrive();
  // Everything above (barriers, TMEM, descriptor prefetch) may have overlapped the previous kernel's
  // tail; from here on its output is read.
  pdl_wait();
  pdl_launch_dependents();
  volatile int* abort_ptr = &abort_flag;
#ifdef KB200_TRACE
  if (blockIdx.x <= 1 && threadIdx.x == 0) marks[2] = clock64();
#endif

  if (warp == 0 || warp == kProducerBWarp) {
    // ---------------- TMA producers ----------------
    // Two threads in two warps, one per operand: issuing a bulk tensor copy costs a lone thread a few
    // hundred cycles, and with narrow tiles that issue time, not the tensor pipe, bounded the K loop.
    // Both wait on the stage's empty barrier and each arrives on its full barrier with its own bytes.
    if (lane == 0) {
      const bool load_a = warp == 0;
      // everything the loop needs in registers: a lone thread pays full latency for every
      // dependent instruction, so the per-slab instruction count is what bounds the issue rate
      const int stages = p.stages, num_units = p.num_units, slab_k = p.slab_k, step_k = p.step_k, kps = p.kps;
      const int bn = p.bn, chunk_n = p.chunk_n, b_mode = p.b_mode, n_chunks = p.n_chunks;
      const uint32_t chunk_bytes = (uint32_t)step_k * kSlabBytes;          // one column chunk of B: step_k rows of 128 bytes
      const uint32_t b_slab_bytes = (uint32_t)bn * kSlabBytes;             // K-major B: one slab of bn rows
      const uint32_t tx_bytes = load_a ? (uint32_t)a_stage_bytes : (uint32_t)b_tile_bytes;
      int s = 0;
      uint32_t wait_parity = 1;                // parity to wait for on the empty barriers of this pass over the ring
      bool ok = true;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x) {
        int tile, ks, batch, tm_i, tn_i, kb_begin, kb_end;
        unit_coords(p, unit, tile, ks, batch, tm_i, tn_i);
        slab_range(p, ks, kb_begin, kb_end);
        const int m0 = tm_i * kTileM, n0 = tn_i * bn;
        const int n0_chunk = tn_i * n_chunks;
        int k_elem = kb_begin * step_k;
        for (int kb = kb_begin; kb < kb_end; ++kb, k_elem += step_k) {
          const uint32_t full = full0 + 8 * s;
          if (!mbar_wait(empty0 + 8 * s, wait_parity, abort_ptr)) {
            if (!*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | 1); *abort_ptr = 1; }
            ok = false;
            break;
          }
          if (load_a) KB200_STAMP(0, tp);
          mbar_expect_tx(full, tx_bytes);
          const uint32_t a_dst = tiles + s * stage_bytes;
          // a slab past the end of K (odd slab count with two slabs per stage) is a box outside the
          // tensor: it arrives as zeros and adds nothing
          if (load_a) {
            for (int j = 0; j < kps; ++j) tma_load_3d(a_dst + j * kATileBytes, &tma_a, full, k_elem + j * slab_k, m0, batch);
          } else if (b_mode == 0) {              // K-major B: one box per slab, like A
            for (int j = 0; j < kps; ++j)
              tma_load_3d(a_dst + a_stage_bytes + j * b_slab_bytes, &tma_b, full, k_elem + j * slab_k, n0, batch);
          } else if (b_mode == 1) {              // N-major B, all column chunks of the tile and all slabs of the stage in one 4-D box
            tma_load_4d(a_dst + a_stage_bytes, &tma_b, full, 0, k_elem, n0_chunk, batch);
          } else {                               // N-major B, N not a multiple of the chunk: one box per chunk
            for (int c = 0; c < n_chunks; ++c)
              tma_load_3d(a_dst + a_stage_bytes + c * chunk_bytes, &tma_b, full, n0 + c * chunk_n, k_elem, batch);
          }
          if (load_a) KB200_STAMP(1, tp);
#ifdef KB200_TRACE
          ++tp;
#endif
          if (++s == stages) { s = 0; wait_parity ^= 1; }
        }
      }
    }
  } else if (warp == 1 || warp == kIssuerBWarp) {
    // ---------------- MMA issuers ----------------
    // One thread issues all MMAs, or (narrow tiles, where the ~62 cycles an MMA instruction costs
    // its issuing thread exceed its tensor time) two threads in two warps issue alternate pipeline
    // stages, each into an accumulator of its own; the epilogue adds the two.
    const int q = warp == 1 ? 0 : 1;
    if (lane == 0 && q < p.issuers) {
      const int nq = p.issuers;
      const int stages = p.stages, splits = p.splits, num_units = p.num_units, bn = p.bn;
      const uint64_t magic_stages = p.magic_stages;
      const uint32_t idesc = p.idesc;
      // descriptors: everything but the 14-bit start address is fixed; advancing along K adds to it
      const uint64_t a_fixed = make_desc(0, 16, 1024);
      const uint64_t b_fixed = p.b_mode == 0 ? make_desc(0, 16, 1024)
                                             : make_desc(0, (uint32_t)(p.step_k * kSlabBytes), (uint32_t)p.b_sbo_bytes, (uint32_t)p.b_layout);
      const uint32_t b_step16 = (p.b_mode == 0 ? 32u : (uint32_t)p.b_step_bytes) >> 4;
      // K-major B keeps its slabs apart (bn rows each); N-major B continues down the rows of its chunks
      const uint32_t b_slab16 = p.b_mode == 0 ? (uint32_t)(p.bn * kSlabBytes) >> 4 : 4u * b_step16;
      const uint32_t tiles16 = tiles >> 4, stage16 = (uint32_t)stage_bytes >> 4, a_tile16 = kATileBytes >> 4;
      const uint32_t a_stage16 = (uint32_t)a_stage_bytes >> 4;
      const uint32_t raw16 = (uint32_t)raw_bytes >> 4;      // from an operand's heads to its tails (exact-FP32 mode)
      constexpr bool split3 = SPLIT3;
      const int kps = p.kps;
      bool ok = true;
      int g0 = 0;          // pipeline steps of this CTA before the current tile: step g uses stage g % stages
      int i = 0;
      for (int unit = blockIdx.x; unit < num_units && ok; unit += gridDim.x, ++i) {
        const int ks = splits > 1 ? unit % splits : 0;
        int kb_begin, kb_end;
        slab_range(p, ks, kb_begin, kb_end);
        const int n_steps = kb_end - kb_begin;
        const int acc = i & 1;
        const uint32_t aph = (i >> 1) & 1;
        // the epilogue must have drained this accumulator (two tiles ago) before it is overwritten
        if (!mbar_wait(tempty0 + 8 * acc, aph ^ 1, abort_ptr)) {
          if (!*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | 4); *abort_ptr = 1; }
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // Exact-FP32 mode: the tensor core truncates every accumulation, an error that grows with the
        // number of MMAs summed into one accumulator (whatever the size of the addend).  The two small
        // products of every step go into an accumulator of their own (at column 0; 2^-11 of the
        // magnitude, so its truncations do not count), and the head x head products of the steps rotate
        // over nacc more; the epilogue adds them all in float32.  The whole allocation is one buffer
        // then: the warps that drain a tile are the ones that prepare the next tile's first stage, so
        // nothing overlaps anyway.
        const int nacc = SPLIT3 ? p.nacc : 1;
        const uint32_t tmem_t = tmem_base + (split3 ? (p.acc2 ? (uint32_t)(acc * 256) : 0u) : (uint32_t)((acc * nq + q) * bn));
        int rot = 0, n_done = 0;
        // this issuer's steps of the tile: the global step numbers congruent to q modulo nq
        // (stage, round) of step g: counted along with one issuer, by multiplication for two
        int g_first = g0 + ((q - g0) & (nq - 1));
        int round = fast_div(g_first, magic_stages);
        int s = g_first - round * stages;
        for (int g = g_first; g < g0 + n_steps; g += nq) {
          // exact-FP32 mode: the stage is ready when the epilogue warps have split it, not when it lands
          if (!mbar_wait((split3 ? split0 : full0) + 8 * s, (uint32_t)round & 1u, abort_ptr)) {
            if (!*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | 2); *abort_ptr = 1; }
            ok = false;
            break;
          }
          if (split3) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (q == 0) KB200_STAMP(2, tm);
          const uint32_t tmem_d = tmem_t + (uint32_t)((rot + (split3 ? 1 : 0)) * bn);
          uint32_t accumulate = n_done >= nacc ? 1u : 0u;
          uint32_t accumulate_small = n_done > 0 ? 1u : 0u;
          if (++rot == nacc) rot = 0;
          ++n_done;
          for (int j = 0; j < kps; ++j) {
            const uint32_t a16 = tiles16 + (uint32_t)s * stage16 + (uint32_t)j * a_tile16;
            const uint32_t b16 = tiles16 + (uint32_t)s * stage16 + a_stage16 + (uint32_t)j * b_slab16;
#pragma unroll
            for (int k = 0; k < kSlabBytes / 32; ++k) {
              // 14-bit start-address field: in a cluster the shared window address carries the CTA rank in
              // its upper bits, which must not spill into the neighbouring descriptor fields
              if (split3) {
                // a*b = (ah + al)(bh + bl) ~ al*bh + ah*bl + ah*bh: the small terms first, al*bl (2^-22 a*b) dropped
                umma(tmem_t, a_fixed | (uint64_t)((a16 + raw16 + 2 * k) & 0x3FFFu), b_fixed | (uint64_t)((b16 + k * b_step16) & 0x3FFFu),
                     idesc, accumulate_small, false);
                umma(tmem_t, a_fixed | (uint64_t)((a16 + 2 * k) & 0x3FFFu), b_fixed | (uint64_t)((b16 + raw16 + k * b_step16) & 0x3FFFu),
                     idesc, 1u, false);
                accumulate_small = 1;
              }
              umma(tmem_d, a_fixed | (uint64_t)((a16 + 2 * k) & 0x3FFFu), b_fixed | (uint64_t)((b16 + k * b_step16) & 0x3FFFu), idesc,
                   accumulate, BF16);
              accumulate = 1;
            }
          }
          umma_commit(empty0 + 8 * s);   // frees the stage once these MMAs have read it
          if (q == 0) KB200_STAMP(3, tm);
#ifdef KB200_TRACE
          ++tm;
#endif
          s += nq;
          if (s >= stages) { s -= stages; ++round; }
        }
        g0 += n_steps;
        if (ok) umma_commit(tfull0 + 8 * acc);   // arrives when every MMA this thread issued for the tile has completed
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // ---------------- epilogue (warps 2..9) ----------------
    // Two warps per TMEM lane quadrant (a warp may only touch lanes 32 * (warp % 4) ..+31); the
    // pair splits the 32-column chunks of the tile between them.
    const int e = warp - 2;
    const int quad = warp & 3;
    const int half = e >> 2;
    float* tbuf = reinterpret_cast<float*>(epi_buf + e * kEpiWarpBytes);
    __nv_bfloat16* stage16 = reinterpret_cast<__nv_bfloat16*>(epi_buf + e * kEpiWarpBytes + kEpiStage16Offset);
    const bool bulk = p.store_mode == 1 && p.splits == 1;
    const bool rowwise = bulk && p.epi_rowwise != 0;
    int sp_s = 0;                 // exact-FP32 mode: the stage these warps split next, and its parity
    uint32_t sp_parity = 0;
    int i = 0;
    bool ok = true;
    // Exact-FP32 mode: before a pipeline step can be multiplied its operands have to be prepared.  Once
    // the copies of a stage have landed, the exact remainder a - head of every float a (head: the 19
    // leading bits, which is all the tensor core reads of the landed float) goes to the second half of
    // the stage; the MMA thread waits for all eight warps.  Steps are taken in the order of the ring.
    auto split_steps = [&](int count) {
      const int n4 = raw_bytes / 16;
      for (int n = 0; n < count; ++n) {
        bool got = mbar_wait(full0 + 8 * sp_s, sp_parity, abort_ptr);
        if (!got && lane == 0 && !*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | 7); *abort_ptr = 1; }
        if (__shfl_sync(0xffffffffu, got ? 1 : 0, 0) == 0 || *abort_ptr) return false;
        float4* head = reinterpret_cast<float4*>(smem_raw + (tiles - raw) + (size_t)sp_s * stage_bytes);
        float4* tail = head + n4;
        for (int idx = e * 32 + lane; idx < n4; idx += kEpiWarps * 32) {
          const float4 v = head[idx];
          float4 t;
          t.x = tf32_tail(v.x);
          t.y = tf32_tail(v.y);
          t.z = tf32_tail(v.z);
          t.w = tf32_tail(v.w);
          tail[idx] = t;
        }
        fence_async_smem();
        // with one accumulator buffer this also orders the warp's reads of the previous tile's
        // accumulators before the MMAs that follow
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(split0 + 8 * sp_s);
        if (++sp_s == p.stages) { sp_s = 0; sp_parity ^= 1u; }
      }
      return true;
    };
    auto steps_of = [&](int unit) {
      int tile, ks, batch, tm_i, tn_i, kb0, kb1;
      unit_coords(p, unit, tile, ks, batch, tm_i, tn_i);
      slab_range(p, ks, kb0, kb1);
      return kb1 - kb0;
    };
    int unsplit = SPLIT3 && (int)blockIdx.x < p.num_units ? steps_of(blockIdx.x) : 0;   // steps of the current tile still to split
    for (int unit = blockIdx.x; unit < p.num_units && ok; unit += gridDim.x, ++i) {
      int tile, ks, batch, tm_i, tn_i;
      unit_coords(p, unit, tile, ks, batch, tm_i, tn_i);
      const int acc = i & 1;
      const uint32_t aph = (i >> 1) & 1;
      const int64_t m0 = (int64_t)tm_i * kTileM, n0 = (int64_t)tn_i * p.bn;
      const int64_t m_first = m0 + quad * 32;
      const bool direct = p.splits == 1;
      int kb_begin_e, kb_end_e;
      slab_range(p, ks, kb_begin_e, kb_end_e);
      const bool two_accumulators = p.issuers == 2 && kb_end_e - kb_begin_e >= 2;   // with one step the second issuer had nothing to do
      // three staging slots per warp fit in the ring, and no later tile of this CTA will refill it
      const bool ring_staging = bulk && unit + (int)gridDim.x >= p.num_units && p.stages * stage_bytes >= kEpiWarps * 3 * kEpiSlotBytes;
      uint8_t* ring_slice = smem_raw + (tiles - raw) + (size_t)e * (3 * kEpiSlotBytes);
      int slot_i = 0;
      float pre_col = 0.0f, pre_mat[32];
      if (direct && !rowwise && n0 + half * 32 < p.mm.N) prefetch_sides(p, pre_col, pre_mat, batch, m_first, n0 + half * 32 + lane);
      // this warp's share of the tile: rows quad*32..+31, column chunks half*32, +64, ...
      // split K: the partial tile goes into this CTA's (now idle) pipeline memory, row-major [128][bn]
      float* part = reinterpret_cast<float*>(smem_raw + (tiles - raw)) + (size_t)(quad * 32) * p.bn;
      // Before its first tile is ready a CTA has nothing for these warps to do, and their code (the
      // unrolled chain, some kilobytes) is not in the instruction cache yet: one dry pass of the loop
      // body over zeros, with nothing stored, takes those misses off the critical path.
      const bool dry_pass = i == 0 && direct && bulk && !KB200_EXPERIMENT(32) && !SPLIT3;
      if (SPLIT3) {
        ok = split_steps(unsplit);
        if (!ok) break;
        // With two accumulator buffers the next tile's first steps are split before this tile is
        // drained, so that its MMAs run under this epilogue; the rest follows after the drain.
        const int next = unit + (int)gridDim.x;
        unsplit = next < p.num_units ? steps_of(next) : 0;
        if (p.acc2 && unsplit > 0) {
          const int ahead = unsplit < p.stages ? unsplit : p.stages;
          ok = split_steps(ahead);
          if (!ok) break;
          unsplit -= ahead;
        }
      }
      for (int c = half * 32 - (dry_pass ? 64 : 0); c < p.bn; c += 64) {
        const bool dry = c < 0;
        if (c == half * 32) {
          bool got = mbar_wait(tfull0 + 8 * acc, aph, abort_ptr);
          if (!got && lane == 0 && !*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | 3); *abort_ptr = 1; }
          ok = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0 && !*abort_ptr;
          if (!ok) break;
#ifdef KB200_TRACE
          if (warp == 2 && lane == 0) { KB200_STAMP(4, te); ++te; }
#endif
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        if (!dry && (n0 + c >= p.mm.N || KB200_EXPERIMENT(16))) break;   // uniform across the warp
        float v[32];
        if (dry) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = 0.0f;
        } else {
          const uint32_t t_addr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)((SPLIT3 ? (p.acc2 ? acc * 256 : 0) : acc * p.issuers * p.bn) + c);
          tmem_ld32(t_addr, v);
          if (SPLIT3) {                  // v holds the small products; the accumulators the K steps rotated over
            const int used = min(p.nacc, kb_end_e - kb_begin_e);
            for (int a = 1; a <= used; ++a) {
              float w[32];
              tmem_ld32(t_addr + (uint32_t)(a * p.bn), w);
#pragma unroll
              for (int j = 0; j < 32; ++j) v[j] += w[j];
            }
          }
          if (two_accumulators) {        // the second issuer's share of the K steps
            float w[32];
            tmem_ld32(t_addr + (uint32_t)p.bn, w);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += w[j];
          }
        }
        if (bulk && !ring_staging) {
          // the bulk stores of the previous block must have read the staging memory before it is rewritten
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
        }
#ifdef KB200_TRACE
        if (warp == 2 && lane == 0 && !dry) { KB200_STAMP(4, te); ++te; }
#endif
        if (!rowwise && direct) {
          // transpose through shared memory: lane = row  ->  lane = column
#pragma unroll
          for (int j = 0; j < 32; ++j) tbuf[lane * 33 + j] = v[j];
          __syncwarp();
#pragma unroll
          for (int r = 0; r < 32; ++r) v[r] = tbuf[r * 33 + lane];
          __syncwarp();
        }
#ifdef KB200_TRACE
        if (warp == 2 && lane == 0 && !dry) { KB200_STAMP(4, te); ++te; }
#endif
        if (direct) {
          // The next block's operands are fetched where their latency hides and no fence waits on them:
          // the per-column value before this block's arithmetic, the matrix operand (whose registers
          // are busy until then) after this block's stores have been issued.
          const bool more = !dry && !rowwise && c + 64 < p.bn && n0 + c + 64 < p.mm.N;
          float next_col = pre_col;
          if (more) prefetch_col(p, next_col, batch, n0 + c + 64 + lane);
          if (rowwise) epilogue_compute_rows(p, v, batch, n0 + (dry ? half * 32 : c));
          else epilogue_compute32(p, v, pre_col, pre_mat, batch, m_first, n0 + (dry ? half * 32 : c) + lane);
          pre_col = next_col;
#ifdef KB200_TRACE
          if (warp == 2 && lane == 0 && !dry) { KB200_STAMP(4, te); ++te; }
#endif
          if (more && !bulk) prefetch_mat(p, pre_mat, batch, m_first, n0 + c + 64 + lane);
          if (bulk) {
            // dense row-major 32 x 32 blocks in shared memory, then one bulk tensor store each: the
            // store engine writes whole 128-byte lines and clips the block at the matrix edges
            uint8_t* sf = reinterpret_cast<uint8_t*>(tbuf);
            uint8_t* sh = reinterpret_cast<uint8_t*>(stage16);
            if (ring_staging && !dry) {
              // last tile of this CTA: the operand ring is idle, so the staging blocks rotate through
              // this warp's slice of it and a store drains while the next blocks are computed
              uint8_t* slot = ring_slice + (size_t)slot_i * kEpiSlotBytes;
              slot_i = slot_i == 2 ? 0 : slot_i + 1;
              sf = slot;
              sh = slot + 4096;
              if (lane == 0) tma_store_wait_read2();
              __syncwarp();
            }
            if (rowwise) stage_rows(sf, sh, v, lane, p.out16 != nullptr);
            else stage_columns(sf, sh, v, lane, p.out16 != nullptr);
            fence_async_smem();
            __syncwarp();
            if (lane == 0 && m_first < p.mm.M && !KB200_EXPERIMENT(1) && !dry) {
              tma_store_3d(&tma_out, smem_u32(sf), (int)(n0 + c), (int)m_first, batch);
              if (p.out16 != nullptr) tma_store_3d(&tma_out16, smem_u32(sh), (int)(n0 + c), (int)m_first, batch);
              tma_store_commit();
            }
            if (more) prefetch_mat(p, pre_mat, batch, m_first, n0 + c + 64 + lane);
          } else {
            epilogue_store32(p, v, batch, m_first, n0 + c + lane);
          }
#ifdef KB200_TRACE
          if (warp == 2 && lane == 0 && !dry) { KB200_STAMP(4, te); ++te; }
#endif
        } else {
          // split K: park this lane's row of the partial tile, eight 128-bit stores whose 16-byte slot
          // within the 32-column group is XORed with the row (no bank conflicts; the reduction undoes it)
          float4* dst = reinterpret_cast<float4*>(part + (size_t)lane * p.bn + c);
#pragma unroll
          for (int q = 0; q < 8; ++q) dst[q ^ (lane & 7)] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
          fence_async_smem();      // the bands are pushed to the neighbours by bulk copies (async proxy)
        }
      }
      // this warp is done reading the accumulator: hand it back to the MMA issuer
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(tempty0 + 8 * acc) : "memory");
#ifdef KB200_TRACE
      if (warp == 2 && lane == 0) { KB200_STAMP(4, te); ++te; }
#endif
    }
    if (bulk && lane == 0) tma_store_wait_read();   // shared memory must outlive the stores that read it
  }

  // ---------------- split K: reduce across the cluster ----------------
  // The `splits` CTAs of a cluster hold partial sums of the same tile, parked row-major in their
  // idle operand rings.  CTA r finishes the band of 128 / splits rows number r: every other CTA
  // PUSHES its part of that band into r's receive area with one bulk shared-to-shared copy that
  // completes on r's `received` barrier -- data and signal in one asynchronous operation, no release
  // fence after the parked tile and no loads over the cluster network (a first version had every
  // CTA announce its parked tile and read the neighbours' bands: the announcing release cost 5500
  // cycles and the scalar remote loads 6000).  r then adds the bands in rank order, its own in its
  // place (so the result does not depend on timing), applies the epilogue and stores.  The hardware
  // cluster barrier, split into arrive and wait, brackets the exchange: nobody pushes before every
  // CTA's barriers exist, nobody leaves before every push out of its shared memory has landed.
  // Every CTA goes through all of it also after an aborted wait: all loops are bounded.
  if (p.splits > 1) {
    const uint32_t received = smem_u32(&bars[2 * kMaxStages + 4]);
    uint32_t rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    const int band_rows = kTileM / p.splits;
    const uint32_t band_bytes = (uint32_t)(band_rows * p.bn * 4);
    const uint32_t recv0 = tiles + (uint32_t)p.recv_offset;
    if (threadIdx.x == 0) mbar_expect_tx(received, (uint32_t)(p.splits - 1) * band_bytes);
    cluster_wait();          // completes the arrive made before the main loop: every CTA's barriers are initialised
    __syncthreads();         // every warp of this CTA has parked its part (and fenced it to the async proxy)
#ifdef KB200_TRACE
    if (blockIdx.x <= 1 && threadIdx.x == 0) marks[3] = clock64();
#endif
    if (lane == 0 && warp < p.splits && warp != (int)rank && !abort_flag) {
      // my partial of band `warp` -> slot `rank` of CTA `warp`'s receive area.  One copy per WARP: issued
      // by the lanes of one warp the seven copies went out one after the other, ~680 cycles each
      // (4760 cycles between the barrier above and the last issue in the cycle stamps).
      const uint32_t dst = map_to_cta(recv0 + rank * band_bytes, (uint32_t)warp);
      const uint32_t bar = map_to_cta(received, (uint32_t)warp);
      asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                   ::"r"(dst), "r"(tiles + (uint32_t)warp * band_bytes), "r"(band_bytes), "r"(bar)
                   : "memory");
    }
#ifdef KB200_TRACE
    if (blockIdx.x <= 1 && warp == kIssuerBWarp && lane == 0) marks[7] = clock64();
#endif
    if (!mbar_wait(received, 0, abort_ptr) && threadIdx.x == 0 && !*abort_ptr) {
      atomicCAS(p.status, 0, (p.kernel_index << 8) | 5);
      *abort_ptr = 1;
    }
    cluster_arrive();        // what this CTA was to receive has landed (or it gave up): see the wait below
#ifdef KB200_TRACE
    if (blockIdx.x <= 1 && threadIdx.x == 0) marks[4] = clock64();
#endif
    if (warp >= 2 && warp < 2 + kEpiWarps && !abort_flag) {
      // The band is small (128 / splits rows): all eight warps walk it as float4 items in row-major
      // order, so every load of a side operand and every store covers whole 128-byte lines, and an
      // item costs a handful of instructions (the 32 x 32 block machinery of the unsplit epilogue took
      // ~5000 cycles for a band that two of the eight warps then handled alone).
      const int e = warp - 2;
      const int unit = blockIdx.x;
      int tile, ks_unused, batch, tm_i, tn_i;
      unit_coords(p, unit, tile, ks_unused, batch, tm_i, tn_i);
      const int64_t m0 = (int64_t)tm_i * kTileM, n0 = (int64_t)tn_i * p.bn;
      const int row_lo = (int)rank * band_rows;
      const int cols4 = p.bn >> 2;
      const int items = band_rows * cols4;
      const uint8_t* const ring = smem_raw + (tiles - raw);
      const MatmulParams& mm = p.mm;
      const DevOperand& out_op = mm.ops[mm.chain.out_slot];
      for (int it = e * 32 + lane; it < items; it += kEpiWarps * 32) {
        const int r = it / cols4, c4 = it - r * cols4;
        const int row = row_lo + r;
        const int64_t m = m0 + row, n = n0 + 4 * c4;
        if (m >= mm.M || n >= mm.N) continue;
        // the parked layout XORs the 16-byte slot within a 32-column group with the row
        const int slot = (c4 & ~7) | ((c4 & 7) ^ (row & 7));
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        for (int sp = 0; sp < p.splits; ++sp) {
          const float4* src = reinterpret_cast<const float4*>(sp == (int)rank ? ring + (size_t)rank * band_bytes
                                                                             : ring + p.recv_offset + (size_t)sp * band_bytes);
          const float4 t = src[r * cols4 + slot];
          v[0] += t.x; v[1] += t.y; v[2] += t.z; v[3] += t.w;
        }
        for (int s = 0; s < mm.chain.n; ++s) {
          const ChainStep st = mm.chain.steps[s];
          float side[4] = {st.imm, st.imm, st.imm, st.imm};
          if (st.slot >= 0) {
            const DevOperand& o = mm.ops[st.slot];
            const float* src = o.ptr + batch * o.stride[0] + m * o.stride[1] + n * o.stride[2];
            if (o.stride[2] == 1 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
              const float4 t = __ldg(reinterpret_cast<const float4*>(src));
              side[0] = t.x; side[1] = t.y; side[2] = t.z; side[3] = t.w;
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) side[j] = __ldg(src + j * o.stride[2]);
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) v[j] = chain_apply_scalar(st.op, v[j], side[j]);
        }
        if (KB200_EXPERIMENT(1)) continue;
        float* dst = out_op.ptr + batch * out_op.stride[0] + m * out_op.stride[1] + n * out_op.stride[2];
        if (out_op.stride[2] == 1 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
          *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) dst[j * out_op.stride[2]] = v[j];
        }
        if (p.out16 != nullptr) {
          __nv_bfloat16* dst16 = p.out16 + batch * out_op.stride[0] + m * out_op.stride[1] + n * out_op.stride[2];
          if (out_op.stride[2] == 1 && (reinterpret_cast<uintptr_t>(dst16) & 7) == 0) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
            uint2 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&lo);
            packed.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(dst16) = packed;
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) dst16[j * out_op.stride[2]] = __float2bfloat16_rn(v[j]);
          }
        }
      }
    }
#ifdef KB200_TRACE
    if (blockIdx.x <= 1 && threadIdx.x == 64) marks[5] = clock64();
#endif
    // every CTA of the cluster has received everything: so every push out of THIS shared memory has landed
    cluster_wait();
#ifdef KB200_TRACE
    if (blockIdx.x <= 1 && threadIdx.x == 0) marks[6] = clock64();
#endif
  }

  // ---------------- common exit ----------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
#ifdef KB200_TRACE
  if (blockIdx.x == 1 && threadIdx.x == 0 && p.splits > 1)
    printf("block1 split phase: entry globaltimer %lld setup_done %lld before cluster sync %lld arrived %lld after %lld reduce done %lld after 2nd sync %lld\n",
           marks[0], marks[2] - marks[1], marks[3] - marks[1], marks[7] - marks[1], marks[4] - marks[1], marks[5] - marks[1], marks[6] - marks[1]);
#endif
#ifdef KB200_TRACE
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    unsigned long long g;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(g));
    printf("KERNEL block0 globaltimer start %lld end %lld (ns) dur %lld | cycles: entry 0 setup_done %lld first_prod %lld exit %lld | units/CTA~%d splits %d num_kb %d bn %d stages %d\n",
           marks[0], (long long)g, (long long)g - marks[0], marks[2] - marks[1], trace[0][0] - marks[1], clock64() - marks[1],
           (p.num_units + (int)gridDim.x - 1) / (int)gridDim.x, p.splits, p.num_kb, p.bn, p.stages);
    if (p.splits > 1) printf("split phase: before cluster sync %lld after %lld warp2 reduce done %lld after 2nd sync %lld (cycles since entry)\n",
           marks[3] - marks[1], marks[4] - marks[1], marks[5] - marks[1], marks[6] - marks[1]);
    const long long t0 = trace[0][0];
    for (int i = 0; i < 160 && i < p.num_kb * 3; ++i)
      printf("slab %3d  prod_wait_done %7lld issued %7lld | mma_full %7lld committed %7lld\n", i, trace[0][i] - t0,
             trace[1][i] - t0, trace[2][i] - t0, trace[3][i] - t0);
    printf("epilogue stamps (tile ready, then per chunk: loaded, transposed, computed, stored; then accumulator released):");
    for (int i = 0; i < 20; ++i) printf(" %lld", trace[4][i] - t0);
    printf("\n");
  }
#endif
  if (abort_flag && threadIdx.x == 0) {
    // give copies that may still be in flight a bounded time to land before shared memory is released
    for (int s = 0; s < p.stages; ++s)
      for (uint32_t i = 0; i < 4096u; ++i)
        if (mbar_try_wait(full0 + 8 * s, 0) || mbar_try_wait(full0 + 8 * s, 1)) break;
  }
  __syncthreads();
  if (warp == 2) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
  }
}

// Strided float32 [batch, rows, cols] (cols contiguous) -> packed bf16 [batch, rows, cols].  Four
// 128-bit loads in flight per thread; all index arithmetic is 32-bit, and a source whose rows and
// batch entries follow each other without gaps is walked as one flat array (64-bit divisions per
// vector made the first version issue-bound: 7.5 us for 6 MB).
__global__ void __launch_bounds__(256) cvt_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                                       int64_t batch, int64_t rows, int64_t cols, int64_t s_batch,
                                                       int64_t s_row) {
  pdl_wait();                 // the producer of this kernel's inputs has completed
  pdl_launch_dependents();    // the next kernel may begin its start-up
  const uint32_t cols4 = (uint32_t)(cols >> 2);
  const uint32_t total = (uint32_t)(batch * rows) * cols4;          // the host keeps this below 2^32
  const bool flat = s_row == cols && (batch == 1 || s_batch == rows * cols);
  const uint32_t step = gridDim.x * blockDim.x;
  constexpr int U = 4;
  for (uint32_t base = blockIdx.x * blockDim.x + threadIdx.x; base < total; base += step * U) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = base + (uint32_t)u * step;
      if (i >= total) continue;
      if (flat) {
        v[u] = *reinterpret_cast<const float4*>(src + (size_t)i * 4);
      } else {
        const uint32_t row = i / cols4, c = i - row * cols4;          // row counts over all batch entries
        const uint32_t bb = row / (uint32_t)rows, r = row - bb * (uint32_t)rows;
        v[u] = *reinterpret_cast<const float4*>(src + (int64_t)bb * s_batch + (int64_t)r * s_row + (size_t)c * 4);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t i = base + (uint32_t)u * step;
      if (i >= total) continue;
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[u].x, v[u].y), hi = __floats2bfloat162_rn(v[u].z, v[u].w);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&lo);
      packed.y = *reinterpret_cast<uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dst + (size_t)i * 4) = packed;
    }
  }
}

// Blocks of 256 threads with four vectors each, at most `cap` blocks.
inline unsigned cvt_grid(int64_t vectors, int64_t cap) {
  const int64_t blocks = (vectors + 1023) / 1024;
  return (unsigned)(blocks < 1 ? 1 : (blocks < cap ? blocks : cap));
}

struct TcState {
  CUtensorMap map_a, map_b;
  CUtensorMap map_out, map_out16;   // bulk-store maps of the output and of its bf16 mirror (store_mode 1)
  TcParams params;
  size_t smem_bytes = 0;
  dim3 grid;
  bool bf16 = false;
  // bf16 operand copies
  __nv_bfloat16* a16 = nullptr;
  __nv_bfloat16* b16 = nullptr;
  bool b_const = false;       // B is a frozen constant: converted once at bind
  bool a_shadow = false;      // A / B is read from the bf16 mirror its producer writes: no conversion launch
  bool b_shadow = false;
  void* pair = nullptr;       // state of the CTA-pair kernel (matmul_pair.cu) when it runs this matmul
};

}  // namespace

bool matmul_wants_bf16_operands(const PlanKernel& k) { return k.desc.precision == KB200_PREC_BF16; }

// Can the tensor-core kernel take this matmul as it stands?
bool tc_eligible(const PlanKernel& k) {
  const kb200_kernel_desc& d = k.desc;
  if (d.precision == KB200_PREC_FP32 && (d.cfg[6] & 1024)) return false;   // config bit 1024: FP32 stays on the CUDA-core kernel (IEEE on non-finite operands)
  if (!k.has_chain) return false;        // any other epilogue DAG runs on the SIMT kernel's tape path
  const DevOperand& A = k.ops[d.a_slot];
  const DevOperand& B = k.ops[d.b_slot];
  if (k.M < 32 || k.N < 64 || k.K < 64) return false;
  // tile indices are divided by multiplication, exact below 2^20 tiles (and every TMA coordinate fits an int)
  if (((k.M + 127) / 128) * ((k.N + 63) / 64) * k.batch >= (int64_t(1) << 20)) return false;
  if (k.N % 4 || k.K % 4) return false;
  if (d.precision == KB200_PREC_BF16 && (k.N % 8 || k.K % 8)) return false;
  // the bf16 conversion pass indexes its vectors with 32 bits
  if (d.precision == KB200_PREC_BF16 && (k.batch * k.M * k.K >= (int64_t(1) << 33) || k.batch * k.K * k.N >= (int64_t(1) << 33))) return false;
  // A: K contiguous; B: N contiguous or K contiguous; 16-byte aligned bases and strides
  if (A.stride[2] != 1) return false;
  const bool b_nmajor = B.stride[2] == 1, b_kmajor = !b_nmajor && B.stride[1] == 1 && B.stride[2] != 0;
  if (!b_nmajor && !b_kmajor) return false;
  if (A.stride[1] % 4 || A.stride[0] % 4 || B.stride[1] % 4 && b_nmajor || B.stride[2] % 4 && b_kmajor || B.stride[0] % 4) return false;
  if (A.stride[1] == 0 || (b_nmajor && B.stride[1] == 0)) return false;
  if (k.batch > 1 && (A.stride[0] == 0 || B.stride[0] == 0)) return false;
  if (!aligned16(A.ptr) || !aligned16(B.ptr)) return false;
  return true;
}

int tc_bind(Plan& plan, PlanKernel& k, int kernel_index) {
  const kb200_kernel_desc& d = k.desc;
  TcState* st = static_cast<TcState*>(k.tc);
  if (!st) {
    st = new TcState();
    k.tc = st;
  }
  st->bf16 = d.precision == KB200_PREC_BF16;
  const int chunk_n = st->bf16 ? 64 : 32, slab_k = st->bf16 ? 64 : 32;
  int bn = d.cfg[1];
  if (bn <= 0) {
    // the widest tile that still gives most SMs a tile of their own (measured: a second, partial
    // wave costs more than narrower tiles); 64 columns when even that leaves SMs idle
    const int64_t tiles_m = (k.M + kTileM - 1) / kTileM;
    bn = 64;
    for (int cand : {256, 128}) {
      if (k.N >= cand && tiles_m * ((k.N + cand - 1) / cand) * k.batch * 5 >= (int64_t)plan.sm_count * 3) {
        bn = cand;
        break;
      }
    }
  }
  const bool split3 = d.precision == KB200_PREC_FP32;     // exact FP32: three TF32 MMAs on split operands
  if (split3 && bn > 128) bn = 128;                        // a stage holds heads and tails of both operands
  if (split3 && d.cfg[1] <= 0 && bn == 64 && k.N >= 128) {
    // Exact-FP32 mode is bound by shared-memory traffic, of which a 128-column tile needs a third less
    // per FLOP: it pays from ~45 tiles on (measured on 768 <- 3072 projections: 48 tiles of 128 columns
    // 66 us against 96 of 64 columns 80 us; but 24 against 48: 64 us against 48 us)
    const int64_t tiles128 = ((k.M + kTileM - 1) / kTileM) * ((k.N + 127) / 128) * k.batch;
    if (tiles128 * 10 >= (int64_t)plan.sm_count * 3) bn = 128;
  }
  if (bn > 256) bn = 256;
  bn = (bn / 64) * 64;                                    // the two epilogue warps of a quadrant take 32 columns each
  if (bn < 64) bn = 64;
  while (bn > 64 && bn / 2 >= k.N) bn /= 2;               // do not make the tile wider than the problem
  (void)chunk_n;
  int stages = d.cfg[3] > 0 ? d.cfg[3] : kMaxStages;   // as deep as shared memory allows: the ring hides ~2000 cycles of TMA latency
  if (stages > kMaxStages) stages = kMaxStages;
  // Two K slabs per stage for narrow tiles: a stage costs the producers and the MMA thread a fixed
  // ~350 cycles of waits and commits on top of 62 per MMA, more than the tensor time of a narrow slab.
  // Two MMA issuers (alternate pipeline steps, an accumulator each) are built in for 64-column tiles,
  // whose MMAs cost more to issue than to execute, but off unless asked for (debug bit 512): they need an
  // even stage count (below), and with the shallower or finer ring that leaves, they measured slower
  // than one issuer with two slabs per stage (k10 of the block: 19.5 against 17.8 us).
  const int issuers = ((d.cfg[6] & 512) && bn <= 64 && !split3) ? 2 : 1;
  // With two issuers one slab per stage (so that the ring can be deep and even), else two for tiles up to 128 columns.
  int kps = d.cfg[2] == 1 || d.cfg[2] == 2 ? d.cfg[2] : (issuers == 2 ? 1 : (bn <= 128 && k.K >= 4 * slab_k ? 2 : 1));
  if (split3) kps = 1;
  const int stage_bytes = (split3 ? 2 : 1) * kps * (kATileBytes + bn * kSlabBytes);
  while (stages > 2 && (size_t)stages * stage_bytes + kEpiBytes + 1024 > (size_t)kMaxDynamicSmem) --stages;
  // Two issuers take alternate pipeline steps.  A wait on an mbarrier tells apart only two consecutive
  // phases, so every stage must belong to ONE issuer, who then sees each of its phases in turn: with an
  // even stage count step g and stage g % stages have the same parity.  (With an odd count ownership
  // alternates, and an issuer a full round ahead takes the phase before last for its own.)
  if (issuers == 2) stages &= ~1;
  TcParams& p = st->params;
  fill_matmul_params(k, &p.mm);
  if (st->bf16) {
    for (int s_i = 0; s_i < p.mm.chain.n; ++s_i) {
      int& op = p.mm.chain.steps[s_i].op;
      if (op == CH_TANH) op = CH_TANH_APPROX;
      else if (op == CH_GELU_TANH) op = CH_GELU_TANH_APPROX;
    }
  }
  p.bn = bn;
  p.stages = stages;
  p.slab_k = slab_k;
  p.kps = kps;
  p.step_k = kps * slab_k;
  p.chunk_n = chunk_n;
  p.num_kb = (int)((k.K + p.step_k - 1) / p.step_k);      // pipeline steps along K
  p.b_step_bytes = (st->bf16 ? 16 : 8) * kSlabBytes;
  // An N-major operand of 32-bit elements must use the 128-byte swizzle on 32-byte atoms, whose
  // pattern repeats every 4 rows; 16-bit elements use the ordinary 128-byte swizzle (8 rows).
  p.b_layout = st->bf16 ? 2 : 1;
  p.b_sbo_bytes = st->bf16 ? 1024 : 512;
  p.b_kmajor = k.ops[d.b_slot].stride[2] == 1 ? 0 : 1;
  p.b_mode = p.b_kmajor ? 0 : (k.N % chunk_n == 0 ? 1 : 2);
  p.debug = d.cfg[6];
  p.issuers = issuers;
  p.split3 = split3 ? 1 : 0;
  p.tmem_cols = 32;
  while (p.tmem_cols < 2 * p.issuers * bn) p.tmem_cols *= 2;   // per issuer two accumulators: the epilogue drains one while the next tile fills the other
  p.nacc = 1;
  p.acc2 = 0;
  if (split3) {
    // all 512 columns, one buffer: an accumulator for the small products and one per 512 of K for the
    // large ones (measured with all three products in one: 6.5e-6 of the largest output per 768 of K,
    // growing in proportion), eight at most; every accumulator costs the epilogue a pass of TMEM loads
    p.tmem_cols = 512;
    const int most = (512 / bn < 8 ? 512 / bn : 8) - 1;   // one is the small products'
    const int64_t want = (k.K + 511) / 512;
    p.nacc = want < 1 ? 1 : (want > most ? most : (int)want);
    p.acc2 = (1 + p.nacc) * bn <= 256 ? 1 : 0;
  }
  p.magic_stages = 0;     // set below, once the stage count is final
  p.tiles_m = (int)((k.M + kTileM - 1) / kTileM);
  p.tiles_n = (int)((k.N + bn - 1) / bn);
  p.num_tiles = p.tiles_m * p.tiles_n * (int)k.batch;
  p.n_chunks = bn / chunk_n;
  p.tiles_per_batch = p.tiles_m * p.tiles_n;
  p.magic_tn = ((uint64_t(1) << 40) + p.tiles_n - 1) / p.tiles_n;
  p.magic_tpb = ((uint64_t(1) << 40) + p.tiles_per_batch - 1) / p.tiles_per_batch;
  // Split K when the tiles alone would leave most SMs idle (128-token projections, the narrow
  // 768-wide layers): every SM then streams a share of the operands.
  int splits = d.cfg[4];
  if (splits <= 0) {
    // Split K over a cluster when the tiles leave SMs idle: the widest split (2, 4, 8) whose CTAs still
    // fit the GPU in one wave with room to place whole clusters (36 clusters of 4 on 148 SMs ran as
    // two waves: 17 us against 10), that leaves every CTA at least three 128-byte slabs of K, and that
    // takes at least 18 slabs off a CTA's serial K loop -- the exchange (park, push the bands, add,
    // store) costs about 3 us, a slab ~0.2 us (measured, TF32: 768 of K over 12 tiles 10.1 -> 7.3 us
    // in eighths, but over 48 tiles 12.5 -> 15.1 us in halves; 3072 of K over 12 tiles 28 -> 9.7 us).
    // In exact-FP32 mode a slab costs three times the MMAs and the operand split: 8 slabs suffice.
    splits = 1;
    const int64_t slabs = (k.K + slab_k - 1) / slab_k;
    for (int cand : {2, 4, 8})
      if ((int64_t)p.num_tiles * cand * 10 <= (int64_t)plan.sm_count * 7 && slabs / cand >= 3 &&
          slabs - slabs / cand >= (split3 ? 8 : 18))
        splits = cand;
  }
  if (splits > p.num_kb) splits = p.num_kb;
  // the reduction runs over a thread-block cluster (<= 8 CTAs) and parks the partial tile in the
  // pipeline's shared memory
  if (splits > 8) splits = 8;
  // split K needs the partial tile to fit the ring, and a receive area of the same size behind the
  // epilogue buffers (tiles up to 128 columns: 64 KB); the ring gives up stages for it, down to two
  if (splits > 1 && bn > 128) splits = 1;
  p.recv_offset = 0;
  if (splits > 1) {
    const size_t tile_bytes = (size_t)kTileM * bn * sizeof(float);
    int fit = stages;
    while (fit > 2 && (size_t)fit * stage_bytes + kEpiBytes + tile_bytes + 1024 > (size_t)kMaxDynamicSmem) --fit;
    if ((size_t)fit * stage_bytes + kEpiBytes + tile_bytes + 1024 > (size_t)kMaxDynamicSmem || (size_t)fit * stage_bytes < tile_bytes) {
      splits = 1;
    } else {
      stages = fit;
      if (issuers == 2) stages &= ~1;
      p.stages = stages;
      p.recv_offset = stages * stage_bytes + kEpiBytes;
    }
  }
  p.splits = splits;
  p.num_units = p.num_tiles * splits;
  p.magic_stages = ((uint64_t(1) << 40) + stages - 1) / stages;
  {
    // step numbers of one CTA are divided by multiplication, exact below 2^20
    const int64_t grid_ctas = splits > 1 ? p.num_units : (p.num_units < plan.sm_count ? p.num_units : plan.sm_count);
    const int64_t steps_per_cta = ((p.num_units + grid_ctas - 1) / grid_ctas) * (int64_t)p.num_kb;
    if (steps_per_cta >= (int64_t(1) << 20))
      return fail(KB200_ERR_UNSUPPORTED, "matmul %s: K loop too long for the tensor-core kernel", d.name);
  }
  // instruction descriptor: D = F32, A/B = TF32 or BF16, A K-major, B MN-major, N = bn, M = 128
  const uint32_t fmt = st->bf16 ? 1u : 2u;
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | (0u << 15) | ((p.b_kmajor ? 0u : 1u) << 16) | ((uint32_t)(bn >> 3) << 17) |
            ((uint32_t)(kTileM >> 4) << 24);
  p.kernel_index = kernel_index;
  p.status = plan.d_status;
  p.out16 = static_cast<__nv_bfloat16*>(k.shadow_out);
  p.pre_col_step = p.pre_mat_step = -1;
  for (int st_i = 0; st_i < k.chain.n; ++st_i) {
    const int slot = k.chain.steps[st_i].slot;
    if (slot < 0) continue;
    const bool per_column = k.ops[slot].stride[1] == 0;
    if (per_column && p.pre_col_step < 0) p.pre_col_step = st_i;
    else if (!per_column && p.pre_mat_step < 0) p.pre_mat_step = st_i;
  }
  st->smem_bytes = (size_t)stages * stage_bytes + kEpiBytes + 1024 + (splits > 1 ? (size_t)kTileM * bn * sizeof(float) : 0);
  // persistent CTAs, one per SM: each walks the tile list with a stride of the grid size
  st->grid = p.splits > 1 ? dim3((unsigned)p.num_units, 1, 1)     // one unit per CTA, clusters of `splits`
                          : dim3((unsigned)(p.num_units < plan.sm_count ? p.num_units : plan.sm_count), 1, 1);

  const DevOperand& A = k.ops[d.a_slot];
  const DevOperand& B = k.ops[d.b_slot];
  const void* a_base = A.ptr;
  const void* b_base = B.ptr;
  // B as a [rows, cols] matrix with cols contiguous: [K, N] when N-major, [N, K] when K-major
  const int64_t b_rows = p.b_kmajor ? k.N : k.K, b_cols = p.b_kmajor ? k.K : k.N;
  int64_t a_row = A.stride[1], a_batch = A.stride[0], b_row = p.b_kmajor ? B.stride[2] : B.stride[1], b_batch = B.stride[0];
  const int64_t b_src_row = b_row;
  k.launches = 1;
  if (st->bf16) {
    if (st->a16) cudaFree(st->a16);
    if (st->b16) cudaFree(st->b16);
    st->a16 = st->b16 = nullptr;
    st->a_shadow = k.a_shadow != nullptr;
    st->b_shadow = k.b_shadow != nullptr;
    if (!st->a_shadow) KB200_CUDA(cudaMalloc(&st->a16, (size_t)k.batch * k.M * k.K * 2));
    if (!st->b_shadow) KB200_CUDA(cudaMalloc(&st->b16, (size_t)k.batch * k.K * k.N * 2));
    st->b_const = d.operands[d.b_slot].base_kind == KB200_BASE_CONST;
    if (st->b_const) {
      const int64_t total = k.batch * b_rows * (b_cols / 4);
      cvt_bf16_kernel<<<cvt_grid(total, 4096), 256>>>(
          B.ptr, st->b16, k.batch, b_rows, b_cols, B.stride[0], b_src_row);
      KB200_CUDA(cudaGetLastError());
      KB200_CUDA(cudaDeviceSynchronize());
    }
    k.launches = 1 + (st->a_shadow ? 0 : 1) + ((st->b_const || st->b_shadow) ? 0 : 1);
    if (st->a_shadow) {
      a_base = k.a_shadow;              // the mirror has the operand's own strides
    } else {
      a_base = st->a16;
      a_row = k.K; a_batch = k.M * k.K;
    }
    if (st->b_shadow) {
      b_base = k.b_shadow;
    } else {
      b_base = st->b16;
      b_row = b_cols; b_batch = k.K * k.N;
    }
  }
  // More than 128 rows: 256-row tiles on SM pairs (matmul_pair.cu) when that kernel covers the epilogue.
  if (st->pair) {
    pair_destroy(st->pair);
    st->pair = nullptr;
  }
  if (pair_eligible(plan, k)) {
    const PairOperands po{st->bf16, a_base, a_row, a_batch, b_base, b_row, b_batch, p.b_kmajor != 0};
    const int rc = pair_bind(plan, k, kernel_index, po, &st->pair);
    if (rc) return rc;
    if (st->pair) return KB200_OK;
  }
  if (!encode_map(&st->map_a, st->bf16, a_base, k.K, k.M, k.batch, a_row, a_batch, slab_k, kTileM, false) ||
      !(p.b_mode == 1 ? encode_map4(&st->map_b, st->bf16, b_base, chunk_n, b_rows, b_cols / chunk_n, k.batch, b_row, b_batch, p.step_k,
                                    bn / chunk_n, !st->bf16)
                      : encode_map(&st->map_b, st->bf16, b_base, b_cols, b_rows, k.batch, b_row, b_batch, p.b_kmajor ? slab_k : chunk_n,
                                   p.b_kmajor ? bn : p.step_k, !st->bf16 && !p.b_kmajor)))
    return fail(KB200_ERR_UNSUPPORTED, "matmul %s: the operands cannot be described to TMA", d.name);
  // Bulk tensor stores need a column-contiguous output with 16-byte aligned base and strides (and the
  // same of the bf16 mirror when there is one); anything else keeps the ordinary stores.
  {
    const DevOperand& O = k.ops[k.chain.out_slot];
    bool ok = d.cfg[7] != 1 && O.stride[2] == 1 && O.stride[1] % 4 == 0 && O.stride[1] >= k.N && aligned16(O.ptr) &&
              (k.batch == 1 || (O.stride[0] % 4 == 0 && O.stride[0] > 0));
    if (ok && p.out16 != nullptr) ok = O.stride[1] % 8 == 0 && (k.batch == 1 || O.stride[0] % 8 == 0) && aligned16(p.out16);
    st->map_out = st->map_a;
    st->map_out16 = st->map_a;
    if (ok) ok = encode_map_store(&st->map_out, false, O.ptr, k.N, k.M, k.batch, O.stride[1], O.stride[0]);
    if (ok && p.out16 != nullptr) ok = encode_map_store(&st->map_out16, true, p.out16, k.N, k.M, k.batch, O.stride[1], O.stride[0]);
    p.store_mode = ok ? 1 : 0;
    // Without a matrix operand in the chain (only immediates and per-column vectors that 128-bit loads
    // can read) the epilogue needs no transpose: a lane keeps its accumulator row.
    bool rowwise = ok && splits == 1 && d.cfg[7] != 2;
    for (int s_i = 0; s_i < k.chain.n && rowwise; ++s_i) {
      const int slot = k.chain.steps[s_i].slot;
      if (slot < 0) continue;
      const DevOperand& o = k.ops[slot];
      rowwise = o.stride[1] == 0 && o.stride[2] == 1 && o.stride[0] % 4 == 0 && aligned16(o.ptr);
    }
    p.epi_rowwise = rowwise ? 1 : 0;
  }
  // The attribute is per function, not per launch: always ask for the ceiling, so that plans with
  // different tile configurations can coexist in one process.
  cudaError_t e = st->bf16 ? cudaFuncSetAttribute(mm_tc_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem)
                  : st->params.split3 ? cudaFuncSetAttribute(mm_tc_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem)
                           : cudaFuncSetAttribute(mm_tc_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem);
  if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(mm_tc_kernel)");
  return KB200_OK;
}

int tc_launch(const Plan& plan, const PlanKernel& k, cudaStream_t s) {
  const TcState* st = static_cast<const TcState*>(k.tc);
  const kb200_kernel_desc& d = k.desc;
  if (st->bf16) {
    const DevOperand& A = k.ops[d.a_slot];
    const DevOperand& B = k.ops[d.b_slot];
    const int64_t cap = (int64_t)plan.sm_count * 8;
    int64_t total = k.batch * k.M * (k.K / 4);
    if (!st->a_shadow)
      KB200_CUDA(launch_kernel(plan.pdl, cvt_bf16_kernel, dim3(cvt_grid(total, cap)),
                               dim3(256), 0, s, (const float*)A.ptr, st->a16, k.batch, k.M, k.K, A.stride[0], A.stride[1]));
    if (!st->b_const && !st->b_shadow) {
      const bool km = st->params.b_kmajor != 0;
      const int64_t rows = km ? k.N : k.K, cols = km ? k.K : k.N;
      total = k.batch * rows * (cols / 4);
      KB200_CUDA(launch_kernel(plan.pdl, cvt_bf16_kernel, dim3(cvt_grid(total, cap)),
                               dim3(256), 0, s, (const float*)B.ptr, st->b16, k.batch, rows, cols, B.stride[0],
                               km ? B.stride[2] : B.stride[1]));
    }
  }
  if (st->pair) return pair_launch(plan, st->pair, s);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = st->grid;
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = st->smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  if (st->params.splits > 1) {
    attr[n_attr].id = cudaLaunchAttributeClusterDimension;
    attr[n_attr].val.clusterDim.x = (unsigned)st->params.splits;
    attr[n_attr].val.clusterDim.y = 1;
    attr[n_attr].val.clusterDim.z = 1;
    ++n_attr;
  }
  if (plan.pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  if (st->bf16) KB200_CUDA(cudaLaunchKernelEx(&cfg, mm_tc_kernel<true, false>, st->map_a, st->map_b, st->map_out, st->map_out16, st->params));
  else if (st->params.split3) KB200_CUDA(cudaLaunchKernelEx(&cfg, mm_tc_kernel<false, true>, st->map_a, st->map_b, st->map_out, st->map_out16, st->params));
  else KB200_CUDA(cudaLaunchKernelEx(&cfg, mm_tc_kernel<false, false>, st->map_a, st->map_b, st->map_out, st->map_out16, st->params));
  KB200_CUDA(cudaGetLastError());
  return KB200_OK;
}

void tc_destroy(PlanKernel& k) {
  TcState* st = static_cast<TcState*>(k.tc);
  if (!st) return;
  if (st->a16) cudaFree(st->a16);
  if (st->b16) cudaFree(st->b16);
  if (st->pair) pair_destroy(st->pair);
  delete st;
  k.tc = nullptr;
}

}  // namespace kb200

// ---------------------------------------------------------------------------------------------
// A matmul entry point that never allocates.
//
// The BF16 tensor-core matmul above needs scratch beyond its inputs and outputs: packed bf16
// copies of both operands, which the plan path obtains with cudaMalloc when buffers are bound.
// Some callers cannot do that -- callers that were handed a fixed memory budget by a serving
// process and may not grow it, hosts that forbid allocation after start-up so that latency stays
// predictable, code that cannot afford the device-wide synchronisation an allocation may imply.  For them the same kernels run here
// with the scratch taken from a fixed array that is part of the library image: every GPU that
// loads libkb200.so holds these bytes from the first use of the library on that device until the
// process exits, whether or not this function is ever called.
// ---------------------------------------------------------------------------------------------

namespace kb200 {
namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;   // 16 MiB in all
constexpr size_t kStaticOperandBytes = kStaticScratchBytes - 256;   // the last 256 bytes hold the status word
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
struct StaticState {
  bool ready = false;
  unsigned char* scratch = nullptr;   // device address of g_static_scratch on this device
};
StaticState g_static_state[kMaxDevices];

// Once per device, with that device current: resolve the device address of the array.  In host
// code the symbol's name is only a handle; the address a kernel may use comes from
// cudaGetSymbolAddress.
std::mutex g_static_mutex;

int static_setup(int device, unsigned char** scratch) {
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (device < 0 || device >= kMaxDevices) return fail(KB200_ERR_ARGUMENT, "kb200_matmul_bf16_static: device %d out of range", device);
  StaticState& st = g_static_state[device];
  if (!st.ready) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static scratch)");
    if (ptr == nullptr || (reinterpret_cast<uintptr_t>(ptr) & 255) != 0)
      return fail(KB200_ERR_CUDA, "kb200_matmul_bf16_static: static scratch resolved to a bad address");
    e = cudaFuncSetAttribute(mm_tc_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxDynamicSmem);
    if (e != cudaSuccess) return cuda_fail(e, "cudaFuncSetAttribute(mm_tc_kernel)");
    st.scratch = static_cast<unsigned char*>(ptr);
    st.ready = true;
  }
  *scratch = st.scratch;
  return KB200_OK;
}

}  // namespace
}  // namespace kb200

extern "C" __attribute__((visibility("default")))
int kb200_matmul_bf16_static(const float* a, const float* b, float* c, int64_t m, int64_t n, int64_t k,
                             int* status_word, void* cuda_stream) {
  using namespace kb200;
  if (a == nullptr || b == nullptr || c == nullptr) return fail(KB200_ERR_ARGUMENT, "kb200_matmul_bf16_static: null operand");
  if (m < 1 || n < 1 || k < 1) return fail(KB200_ERR_ARGUMENT, "kb200_matmul_bf16_static: sizes must be positive");
  if (n < 64 || k < 64 || n % 8 || k % 8)
    return fail(KB200_ERR_UNSUPPORTED, "kb200_matmul_bf16_static: needs n, k >= 64 and multiples of 8 (got n=%lld k=%lld)",
                (long long)n, (long long)k);
  if (!aligned16(a) || !aligned16(b) || !aligned16(c))
    return fail(KB200_ERR_UNSUPPORTED, "kb200_matmul_bf16_static: operands must be 16-byte aligned");
  const uint64_t a_bytes = (uint64_t)m * k * 2, b_bytes = (uint64_t)k * n * 2;
  const uint64_t b_offset = (a_bytes + 255) & ~uint64_t(255);
  if (m > (int64_t(1) << 24) || n > (int64_t(1) << 24) || k > (int64_t(1) << 24) || b_offset + b_bytes > kStaticOperandBytes)
    return fail(KB200_ERR_ARGUMENT,
                "kb200_matmul_bf16_static: operands need %llu bytes of bf16 scratch, the static array holds %llu "
                "(limit: 2*(m*k + k*n) bytes, each operand rounded up to 256, <= 16 MiB - 256); use the plan "
                "interface for larger shapes",
                (unsigned long long)(b_offset + b_bytes), (unsigned long long)kStaticOperandBytes);
  int device = 0;
  KB200_CUDA(cudaGetDevice(&device));
  unsigned char* scratch = nullptr;
  int rc = static_setup(device, &scratch);
  if (rc) return rc;
  __nv_bfloat16* a16 = reinterpret_cast<__nv_bfloat16*>(scratch);
  __nv_bfloat16* b16 = reinterpret_cast<__nv_bfloat16*>(scratch + b_offset);

  int bn = 128;
  while (bn > 64 && bn / 2 >= n) bn /= 2;
  const int stages = 4, slab_k = 64, chunk_n = 64;
  TcParams p{};
  p.mm.batch = 1; p.mm.M = m; p.mm.N = n; p.mm.K = k;
  p.mm.a_slot = 0; p.mm.b_slot = 1; p.mm.n_operands = 3; p.mm.has_chain = 1;
  p.mm.ops[2].ptr = c;
  p.mm.ops[2].stride[0] = 0; p.mm.ops[2].stride[1] = n; p.mm.ops[2].stride[2] = 1;
  p.mm.chain.n = 0; p.mm.chain.first_slot = -1; p.mm.chain.out_slot = 2;
  p.bn = bn; p.stages = stages; p.slab_k = slab_k; p.chunk_n = chunk_n;
  p.kps = 1; p.step_k = slab_k;
  p.issuers = 1;
  p.split3 = 0;
  p.nacc = 1;
  p.acc2 = 0;
  p.magic_stages = ((uint64_t(1) << 40) + stages - 1) / stages;
  p.num_kb = (int)((k + slab_k - 1) / slab_k);
  p.b_step_bytes = 16 * kSlabBytes;
  p.b_layout = 2; p.b_sbo_bytes = 1024;
  p.b_kmajor = 0;
  p.b_mode = 2;
  p.tmem_cols = 32;
  while (p.tmem_cols < 2 * bn) p.tmem_cols *= 2;
  p.tiles_m = (int)((m + kTileM - 1) / kTileM);
  p.tiles_n = (int)((n + bn - 1) / bn);
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.n_chunks = bn / chunk_n;
  p.tiles_per_batch = p.num_tiles;
  p.magic_tn = ((uint64_t(1) << 40) + p.tiles_n - 1) / p.tiles_n;
  p.magic_tpb = ((uint64_t(1) << 40) + p.tiles_per_batch - 1) / p.tiles_per_batch;
  p.splits = 1;
  p.num_units = p.num_tiles;
  p.pre_col_step = p.pre_mat_step = -1;
  p.out16 = nullptr;
  p.idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
  p.kernel_index = 0;
  cudaStream_t s = static_cast<cudaStream_t>(cuda_stream);
  if (status_word != nullptr) {
    p.status = status_word;
  } else {
    // The array keeps what the last call left in it.  Only the status word has to start at zero.
    p.status = reinterpret_cast<int*>(scratch + kStaticOperandBytes);
    KB200_CUDA(cudaMemsetAsync(p.status, 0, sizeof(int), s));
  }
  CUtensorMap map_a, map_b;
  if (!encode_map(&map_a, true, a16, k, m, 1, k, m * k, slab_k, kTileM, false) ||
      !encode_map(&map_b, true, b16, n, k, 1, n, k * n, chunk_n, slab_k, false))
    return fail(KB200_ERR_UNSUPPORTED, "kb200_matmul_bf16_static: the operands cannot be described to TMA");
  const int64_t cap = 148 * 8;
  int64_t total = m * (k / 4);
  cvt_bf16_kernel<<<cvt_grid(total, cap), 256, 0, s>>>(a, a16, 1, m, k, 0, k);
  total = k * (n / 4);
  cvt_bf16_kernel<<<cvt_grid(total, cap), 256, 0, s>>>(b, b16, 1, k, n, 0, n);
  const size_t smem = (size_t)stages * (kATileBytes + bn * kSlabBytes) + kEpiBytes + 1024;
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  dim3 grid((unsigned)(p.num_tiles < sms ? p.num_tiles : sms), 1, 1);
  p.store_mode = 0;   // ordinary stores: the two store maps are unused placeholders
  p.epi_rowwise = 0;
  mm_tc_kernel<true, false><<<grid, kThreads, smem, s>>>(map_a, map_b, map_a, map_a, p);
  KB200_CUDA(cudaGetLastError());
  return KB200_OK;
}


// Reads back the status word that calls with status_word == NULL use on the current device (a
// blocking 4-byte copy: call it after synchronising with the stream the matmul ran on).
extern "C" __attribute__((visibility("default")))
int kb200_matmul_bf16_static_status(void) {
  using namespace kb200;
  int device = 0;
  KB200_CUDA(cudaGetDevice(&device));
  unsigned char* scratch = nullptr;
  int rc = static_setup(device, &scratch);
  if (rc) return rc;
  int word = 0;
  KB200_CUDA(cudaMemcpy(&word, scratch + kStaticOperandBytes, sizeof(int), cudaMemcpyDeviceToHost));
  if (word != 0)
    return fail(KB200_ERR_DEVICE_WAIT, "kb200_matmul_bf16_static: a bounded device-side wait ran out (code 0x%x, site %d)", word, word & 0xff);
  return KB200_OK;
}
