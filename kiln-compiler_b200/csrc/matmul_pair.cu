// CTA-pair tensor-core matmul for sm_100a: 256 x BN output tiles computed by the two SMs of a
// thread-block cluster with tcgen05.mma.cta_group::2.  Same role as matmul_tc.cu (the reference's
// matmul generator with a fused epilogue, kiln/gpu/codegen.py:484-530, 563-598) for problems with
// more than 128 rows in the TF32 and BF16 operand modes.
//
// Why pairs: one issuing thread drives the tensor cores of two SMs, every CTA stages only its own
// half of the B tile (half the shared-memory fill and half the B bytes per FLOP of a 128-row
// tile), and a 256 x 128 tile keeps each MMA instruction at 64 tensor cycles per SM, above the
// ~62 cycles an instruction occupies the pipe whatever its width.
//
// A cluster is two CTAs (ranks 0 = leader, 1 = peer), one per SM, persistent over a static list
// of tiles.  Per CTA, 512 threads:
//   warp 0      TMA producer (one lane): its CTA's 128 rows of A and its half of the B columns per
//               pipeline stage, plain (non-multicast) bulk tensor loads with .cta_group::2 so that
//               both CTAs' bytes complete on the LEADER's `full` barrier.
//   warp 1      TMEM allocation (both CTAs execute the .cta_group::2 alloc / dealloc); then, leader
//               only, the MMA issuer (one lane): tcgen05.mma.cta_group::2 (M = 256, N = BN) reads both
//               CTAs' stages and writes each CTA's 128 accumulator rows into that CTA's TMEM; one
//               multicast tcgen05.commit hands the stage back to both CTAs (`empty`) or the
//               accumulator on (`tfull`).
//   warps 2-13  epilogue of the CTA's own 128 rows, three warps per TMEM lane quadrant: tcgen05.ld
//               of a 32-column block, the fused chain with a lane per accumulator row, the block
//               staged in the warp's shared-memory slot and written by bulk tensor stores, float32
//               and / or the bf16 mirror.  A full-matrix operand of the chain (residual, mask) is
//               brought into the slot by a bulk tensor LOAD, so no warp ever gathers rows from
//               global memory.  Accumulators are double buffered in TMEM: the epilogue of tile i
//               runs under the main loop of tile i + 1; both CTAs' warps release the buffer on the
//               leader's `tempty` barrier.  (Warps 14 and 15 are idle: 512 threads are what leaves
//               the compiler 128 registers per thread.)
// Every mbarrier wait is bounded: on expiry the thread records (kernel, site) in the plan's status
// word, raises its CTA's abort flag, all roles fall through to the exit, which passes the cluster
// barrier (every path reaches it), frees TMEM and returns.  The other CTA's waits run out by themselves.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cstdio>
#include <cstdlib>

#include "device_math.cuh"
#include "kb200_internal.h"
#include "matmul.h"
#include "matmul_pair.h"
#include "tc_common.cuh"
#include "tc_epilogue.cuh"

namespace kb200 {

namespace {

using namespace tc;

constexpr int kPairThreads = 512;
constexpr int kPairEpiWarps = 12;
constexpr int kPairFirstEpiWarp = 2;
constexpr int kPairWarpsPerQuad = kPairEpiWarps / 4;
constexpr int kPairBlocksPerWarp = (8 + kPairWarpsPerQuad - 1) / kPairWarpsPerQuad;   // 32-column blocks of a 256-column tile
constexpr int kPairMaxStages = 8;
constexpr int kPairATileBytes = 128 * 128;        // 128 rows x one 128-byte K slab
#ifdef KB200_TRACE
constexpr int kPairSmemCeiling = 200 * 1024;      // the trace arrays take static shared memory
#define PAIR_STAMP(role, idx) do { if (blockIdx.x <= 1 && (idx) < 128) trace[role][idx] = clock64(); } while (0)
#else
constexpr int kPairSmemCeiling = 225 * 1024;      // opt-in ceiling, the same for every launch of the kernel
#define PAIR_STAMP(role, idx) do { } while (0)
#endif
// barrier indices
constexpr int kBarFull = 0, kBarEmpty = kPairMaxStages, kBarTFull = 2 * kPairMaxStages, kBarTEmpty = kBarTFull + 2,
              kBarRes = kBarTEmpty + 2, kBarCount = kBarRes + kPairEpiWarps;

enum : int { SIDE_NONE = 0, SIDE_IMM = 1, SIDE_COL = 2, SIDE_RES = 3 };

struct PairStep {
  int op;                // ChainOp
  int kind;              // SIDE_*
  float imm;
  const float* ptr;      // SIDE_COL: one value per column, contiguous
  int64_t batch_stride;  // SIDE_COL: elements between batch entries
};

struct PairParams {
  // what the producer and the MMA thread need comes first (constant-bank lines touched at start-up)
  int bn, half_bn, stages, num_kb, slab_k, kps, step_k;
  int b_kmajor;          // B is [N, K] with K contiguous (boxes like A); else [K, N], one 4-D box per stage
  int chunk_n;           // columns per 128-byte row of an N-major B chunk: 32 (tf32) or 64 (bf16)
  uint32_t b_lbo_bytes, b_sbo_bytes, b_layout, b_step16, b_slab16;
  uint32_t idesc;
  int tmem_cols;
  int tiles_n, tiles_per_batch, num_tiles;
  uint64_t magic_tn, magic_tpb;
  int kernel_index;
  int* status;
  // epilogue
  int64_t M, N;
  __nv_bfloat16* out16;  // bf16 mirror of the output (same strides), or null
  int store32;           // 0: only the mirror is stored (every reader of this output takes the mirror)
  int slots, slot_bytes;
  int res_step;          // chain step whose operand arrives by bulk tensor load, or -1
  int res_batched;       // that operand has one matrix per batch entry (else the same for all)
  int n_steps;
  PairStep steps[kMaxChain];
#ifdef KB200_TRACE
  int debug;             // experiments of the trace build: 1 no bulk stores, 2 no staging, 4 no tensor-memory loads
#endif
};

__device__ __forceinline__ int pair_div(int x, uint64_t magic) { return (int)(((uint64_t)(uint32_t)x * magic) >> 40); }

__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
template <bool BF16>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (BF16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
// Arrives, when every MMA issued so far by this thread has completed, on the mbarrier at this offset
// in BOTH CTAs of the pair (a commit, not a copy: the arrival is what is sent to the two CTAs).  One
// instruction: a commit costs the issuing thread about as much as two MMAs.
__device__ __forceinline__ void umma_pair_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(bar), "h"((uint16_t)3)
               : "memory");
}
__device__ __forceinline__ uint32_t ld_cluster_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
// At most `allowed` of this thread's most recent bulk-store groups may still be reading shared memory.
__device__ __forceinline__ void store_wait_read(int allowed) {
  switch (allowed) {
    case 0: asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory"); break;
    default: asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory"); break;
  }
}

template <bool BF16, int KPS>
__global__ void __launch_bounds__(kPairThreads, 1)
mm_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const __grid_constant__ CUtensorMap tma_out, const __grid_constant__ CUtensorMap tma_out16,
               const __grid_constant__ CUtensorMap tma_res, const __grid_constant__ PairParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bars[kBarCount];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ PairStep chain_steps[kMaxChain];     // looked up by a run-time index for every block
#ifdef KB200_TRACE
  __shared__ long long trace[5][128];
  __shared__ long long marks[8];
  int tp = 0, tq = 0, te = 0;
  if (blockIdx.x <= 1 && threadIdx.x == 0) marks[0] = clock64();
#endif

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;     // the 128-byte swizzle pattern repeats every 1024 bytes
  const int a_stage_bytes = KPS * kPairATileBytes;
  const int b_stage_bytes = KPS * p.half_bn * 128;
  const int stage_bytes = a_stage_bytes + b_stage_bytes;
  const uint32_t epi_base = tiles + (uint32_t)(p.stages * stage_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint32_t rank;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const uint32_t full0 = smem_u32(&bars[kBarFull]), empty0 = smem_u32(&bars[kBarEmpty]);
  const uint32_t tfull0 = smem_u32(&bars[kBarTFull]), tempty0 = smem_u32(&bars[kBarTEmpty]);

  if (threadIdx.x == 32) {
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
    prefetch_tensormap(&tma_out);
    if (p.out16 != nullptr) prefetch_tensormap(&tma_out16);
    if (p.res_step >= 0) prefetch_tensormap(&tma_res);
  }
  if (warp == 0) {
    if (lane == 0) abort_flag = 0;
    for (int b = lane; b < kBarCount; b += 32)
      mbar_init(full0 + 8 * b, b >= kBarTEmpty && b < kBarRes ? 2 * kPairEpiWarps : 1);   // both CTAs' epilogue warps release an accumulator
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // The parameter block is read through the constant cache, cold at kernel start: touch the lines the
  // producer and the MMA thread need now, under the set-up, instead of in front of the first copy.
  // Both CTAs' barriers must exist before either signals the other: arrive on the cluster barrier as
  // soon as this CTA's are initialised, wait for it after the TMEM allocation below.
  cluster_arrive();
  if (lane == 0 && warp < 2)
    asm volatile("" ::"r"(p.bn), "r"(p.idesc), "r"(p.num_tiles), "l"(p.magic_tn), "l"(p.magic_tpb), "l"(p.status) : "memory");
  if (warp == 2 && lane < kMaxChain) chain_steps[lane] = p.steps[lane];
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)),
                 "r"((uint32_t)p.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_slot;
#ifdef KB200_TRACE
  if (blockIdx.x <= 1 && threadIdx.x == 0) marks[1] = clock64();
#endif
  cluster_wait();
#ifdef KB200_TRACE
  if (blockIdx.x <= 1 && threadIdx.x == 0) marks[2] = clock64();
#endif
  volatile int* abort_ptr = &abort_flag;
  // The MMA instruction names one TMEM address for both CTAs: the two allocations must agree.
  if (threadIdx.x == 0 && rank == 1) {
    const uint32_t leader_base = ld_cluster_u32(map_to_cta(smem_u32(&tmem_base_slot), 0));
    if (leader_base != tmem_base) {
      atomicCAS(p.status, 0, (p.kernel_index << 8) | 9);
      *abort_ptr = 1;
    }
  }
  // Everything above may have overlapped the previous kernel's tail; from here on its output is read.
  pdl_wait();
  pdl_launch_dependents();
#ifdef KB200_TRACE
  if (blockIdx.x <= 1 && threadIdx.x == 0) marks[3] = clock64();
#endif

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      const int stages = p.stages, num_tiles = p.num_tiles, num_kb = p.num_kb, slab_k = p.slab_k, step_k = p.step_k;
      constexpr int kps = KPS;
      const int bn = p.bn, half_bn = p.half_bn, b_kmajor = p.b_kmajor, chunk_n = p.chunk_n;
      const uint32_t tx_bytes = (uint32_t)stage_bytes;
      const uint32_t full_leader0 = map_to_cta(full0, 0);
      int s = 0;
      uint32_t wait_parity = 1;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int batch = pair_div(tile, p.magic_tpb);
        const int rem = tile - batch * p.tiles_per_batch;
        const int tm_i = pair_div(rem, p.magic_tn);
        const int tn_i = rem - tm_i * p.tiles_n;
        const int m_row = tm_i * 256 + (int)rank * 128;
        const int n_col = tn_i * bn + (int)rank * half_bn;
        int k_elem = 0;
        for (int kb = 0; kb < num_kb; ++kb, k_elem += step_k) {
          if (!mbar_wait_cluster(empty0 + 8 * s, wait_parity, abort_ptr)) {
            if (!*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | 1); *abort_ptr = 1; }
            ok = false;
            break;
          }
          // the leader's barrier counts the bytes of both CTAs (the peer's may land first: the phase
          // cannot complete before this arrival)
          PAIR_STAMP(0, tp);
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * tx_bytes);
          const uint32_t bar = full_leader0 + 8 * s;
          const uint32_t dst = tiles + (uint32_t)(s * stage_bytes);
          for (int j = 0; j < kps; ++j) tma_load_3d_pair(dst + j * kPairATileBytes, &tma_a, bar, k_elem + j * slab_k, m_row, batch);
          if (b_kmajor) {
            for (int j = 0; j < kps; ++j)
              tma_load_3d_pair(dst + a_stage_bytes + j * half_bn * 128, &tma_b, bar, k_elem + j * slab_k, n_col, batch);
          } else {
            tma_load_4d_pair(dst + a_stage_bytes, &tma_b, bar, 0, k_elem, n_col / chunk_n, batch);
          }
          PAIR_STAMP(1, tp);
#ifdef KB200_TRACE
          ++tp;
#endif
          if (++s == stages) { s = 0; wait_parity ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (leader CTA) ----------------
    // A lone thread pays full latency for every instruction: ~60 cycles per tcgen05.mma, ~100 per
    // commit, whatever the tile size.  So a step is one barrier probe, 4 * KPS MMAs whose descriptor
    // words advance by additions, and ONE commit for both CTAs.
    if (lane == 0 && rank == 0) {
      const int stages = p.stages, num_tiles = p.num_tiles, num_kb = p.num_kb, bn = p.bn;
      const uint32_t idesc = p.idesc;
      const uint64_t a_fixed = make_desc(0, 16, 1024);
      const uint64_t b_fixed = p.b_kmajor ? make_desc(0, 16, 1024) : make_desc(0, p.b_lbo_bytes, p.b_sbo_bytes, p.b_layout);
      const uint32_t a_hi = (uint32_t)(a_fixed >> 32), b_hi = (uint32_t)(b_fixed >> 32);
      const uint32_t a_lo_fixed = (uint32_t)a_fixed, b_lo_fixed = (uint32_t)b_fixed;   // the bits of the low word above the start address
      const uint32_t b_step16 = p.b_step16, b_slab16 = p.b_slab16;
      // start addresses (16-byte units, 14 bits: the CTA rank in the upper bits of a cluster's shared
      // window address must not spill into the neighbouring fields) of stage 0
      const uint32_t a_first = (tiles >> 4) & 0x3FFFu, stage16 = (uint32_t)stage_bytes >> 4;
      const uint32_t b_first = a_first + ((uint32_t)a_stage_bytes >> 4);
      int s = 0, i = 0;
      uint32_t parity = 0, a16 = a_first, b16 = b_first;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++i) {
        const int acc = i & 1;
        const uint32_t aph = (i >> 1) & 1;
        // both CTAs' epilogue warps have drained this accumulator (two tiles ago)
        if (!mbar_wait_cluster(tempty0 + 8 * acc, aph ^ 1, abort_ptr)) {
          if (!*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | 4); *abort_ptr = 1; }
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(acc * bn);
        uint32_t accumulate = 0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full0 + 8 * s, parity, abort_ptr)) {
            if (!*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | 2); *abort_ptr = 1; }
            ok = false;
            break;
          }
          PAIR_STAMP(2, tq);
#ifdef KB200_TRACE
          long long fine[6];
          fine[0] = clock64();
#endif
#pragma unroll
          for (int j = 0; j < KPS; ++j) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint64_t adesc = ((uint64_t)a_hi << 32) | (a_lo_fixed | ((a16 + (uint32_t)(j * (kPairATileBytes >> 4) + 2 * k)) & 0x3FFFu));
              const uint64_t bdesc = ((uint64_t)b_hi << 32) | (b_lo_fixed | ((b16 + (uint32_t)j * b_slab16 + (uint32_t)k * b_step16) & 0x3FFFu));
#ifdef KB200_TRACE
              if (!(p.debug & 32))
#endif
              umma_pair<BF16>(tmem_d, adesc, bdesc, idesc, accumulate);
              accumulate = 1;
#ifdef KB200_TRACE
              if (j == 0) fine[1 + k] = clock64();
#endif
            }
          }
          // the stage is free in both CTAs once these MMAs have read it
          umma_pair_commit(empty0 + 8 * s);
#ifdef KB200_TRACE
          fine[5] = clock64();
          (void)fine;
#endif
          PAIR_STAMP(3, tq);
#ifdef KB200_TRACE
          ++tq;
#endif
          a16 += stage16;
          b16 += stage16;
          if (++s == stages) { s = 0; parity ^= 1; a16 = a_first; b16 = b_first; }
        }
        if (ok) umma_pair_commit(tfull0 + 8 * acc);
      }
    }
  } else if (warp >= kPairFirstEpiWarp && warp < kPairFirstEpiWarp + kPairEpiWarps) {
    // ---------------- epilogue (warps 2..17) ----------------
    // Four warps per TMEM lane quadrant (a warp may only touch lanes 32 * (warp % 4) ..+31); warp g of a
    // quadrant takes the 32-column blocks g, g + 4 of the tile.  Sixteen warps, because the epilogue is
    // bound by instruction issue and by the latencies inside a pass (tensor-memory load, the wait for
    // the slot's last store, the proxy fence): with two warps per scheduler the schedulers issued in
    // 46 % of the cycles, a probe of independent multiply-adds in 90 %.
    const int e = warp - kPairFirstEpiWarp, quad = warp & 3, group = e >> 2;
    const int slot_bytes = p.slot_bytes;
    const uint32_t slot0 = epi_base + (uint32_t)(e * slot_bytes);
    uint8_t* const slot0_ptr = smem_raw + (slot0 - raw);
    const uint32_t res_bar = smem_u32(&bars[kBarRes + e]);
    const uint32_t tempty_leader0 = map_to_cta(tempty0, 0);
    const bool has_res = p.res_step >= 0, with16 = p.out16 != nullptr, with32 = p.store32 != 0;
    // where the block's per-column operand passes through shared memory (-1: broadcast by shuffles)
    const int scratch_off = !has_res ? 0 : (with16 ? 4096 : -1);
    const int n_steps = p.n_steps;
    int col_step = -1;
    for (int s = 0; s < n_steps && col_step < 0; ++s)
      if (chain_steps[s].kind == SIDE_COL) col_step = s;
    float col_pre[kPairBlocksPerWarp];
#pragma unroll
    for (int j = 0; j < kPairBlocksPerWarp; ++j) col_pre[j] = 0.0f;
    uint32_t res_phase = 0;
    bool ok = true;
    int i = 0;
    bool dry = true;               // the rehearsal pass described at the tile loop
    // The fused chain on one 32 x 32 block held a lane per row (v[q] = column n + q of this lane's row).
    auto run_chain = [&](float (&v)[32], float mine, int n, int batch) {
      for (int s = 0; s < n_steps; ++s) {
        const PairStep st = chain_steps[s];
        float side[32];
        if (st.kind == SIDE_RES) {
          if (!dry) {
            bool landed = mbar_wait(res_bar, res_phase, abort_ptr);
            if (!landed && !*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | 5); *abort_ptr = 1; }
            res_phase ^= 1u;
          }
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 t = *reinterpret_cast<const float4*>(slot0_ptr + lane * 128 + ((q ^ (lane & 7)) << 4));
            side[4 * q] = t.x; side[4 * q + 1] = t.y; side[4 * q + 2] = t.z; side[4 * q + 3] = t.w;
          }
        } else if (s == col_step && scratch_off >= 0) {
          const float4* col_smem = reinterpret_cast<const float4*>(slot0_ptr + scratch_off);
#pragma unroll
          for (int q = 0; q < 8; ++q) {        // every lane reads the same 16 bytes: a broadcast
            const float4 t = col_smem[q];
            side[4 * q] = t.x; side[4 * q + 1] = t.y; side[4 * q + 2] = t.z; side[4 * q + 3] = t.w;
          }
        } else if (s == col_step) {
#pragma unroll
          for (int q = 0; q < 32; ++q) side[q] = __shfl_sync(0xffffffffu, mine, q);
        } else if (st.kind == SIDE_COL) {
          const float4* base = reinterpret_cast<const float4*>(st.ptr + (int64_t)batch * st.batch_stride + n);
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const float4 t = n + 4 * q < p.N ? __ldg(base + q) : make_float4(0.f, 0.f, 0.f, 0.f);
            side[4 * q] = t.x; side[4 * q + 1] = t.y; side[4 * q + 2] = t.z; side[4 * q + 3] = t.w;
          }
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q) side[q] = st.imm;
        }
        chain_step32(st.op, v, side);
      }
    };
    // The first pass over the loop body is a rehearsal: while the first tile is still being multiplied
    // the warp runs one block of the same instructions on whatever tensor memory holds, waits for
    // nothing, requests nothing and stores nothing.  The kernel's code is cold at every launch, and the
    // instruction-cache misses of the first real epilogue would otherwise hold back the accumulator the
    // main loop needs two tiles later.
    for (int tile = pair; tile < p.num_tiles && ok;) {
      const int batch = pair_div(tile, p.magic_tpb);
      const int rem = tile - batch * p.tiles_per_batch;
      const int tm_i = pair_div(rem, p.magic_tn);
      const int tn_i = rem - tm_i * p.tiles_n;
      const int acc = dry ? 1 : (i & 1);
      const uint32_t aph = (i >> 1) & 1;
      const int m_first = tm_i * 256 + (int)rank * 128 + quad * 32;
      const int n0 = tn_i * p.bn;
      const bool rows_ok = m_first < p.M;
      // the first per-column operand of the chain (a bias) is fetched for this warp's blocks before the
      // accumulator is ready: lane l holds column l of each block, one coalesced 128-byte load per block
      if (col_step >= 0 && rows_ok) {
        const float* src = chain_steps[col_step].ptr + (int64_t)batch * chain_steps[col_step].batch_stride + n0 + lane;
#pragma unroll
        for (int j = 0; j < kPairBlocksPerWarp; ++j) {
          const int c = 32 * (group + kPairWarpsPerQuad * j);
          col_pre[j] = (c < p.bn && n0 + c + lane < p.N) ? __ldg(src + c) : 0.0f;
        }
      }
      // the first block's matrix operand is requested before the accumulator is ready
      bool res_ready = false;
      if (has_res && !dry && rows_ok && 32 * group < p.bn && n0 + 32 * group < p.N) {
        if (lane == 0) {
          store_wait_read(0);
          mbar_expect_tx(res_bar, 4096);
          tma_load_3d(slot0, &tma_res, res_bar, n0 + 32 * group, m_first, p.res_batched ? batch : 0);
        }
        res_ready = true;
      }
      if (!dry) {
        bool got = mbar_wait_cluster_relaxed(tfull0 + 8 * acc, aph, abort_ptr);
        if (!got && lane == 0 && !*abort_ptr) { atomicCAS(p.status, 0, (p.kernel_index << 8) | 3); *abort_ptr = 1; }
        ok = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0 && !*abort_ptr;
        if (!ok) break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#ifdef KB200_TRACE
      if (warp == 4 && lane == 0) { PAIR_STAMP(4, te); ++te; }
#endif
#pragma unroll 1
      for (int j = 0; j < kPairBlocksPerWarp; ++j) {
        const int c = 32 * (group + kPairWarpsPerQuad * j);
        const int n = n0 + c;
        if (c >= p.bn || !rows_ok || n >= p.N) break;          // uniform across the warp
        float mine = col_pre[0];
#pragma unroll
        for (int q = 1; q < kPairBlocksPerWarp; ++q)
          if (j == q) mine = col_pre[q];
        // the slot's last bulk stores have finished reading it
        if (lane == 0) store_wait_read(0);
        __syncwarp();
        // a full-matrix operand of the chain (residual, mask) is brought INTO the slot by a bulk tensor
        // load, under the tensor-memory load below
        if (has_res && !dry && !(j == 0 && res_ready) && lane == 0) {
          mbar_expect_tx(res_bar, 4096);
          tma_load_3d(slot0, &tma_res, res_bar, n, m_first, p.res_batched ? batch : 0);
        }
        if (col_step >= 0 && scratch_off >= 0) reinterpret_cast<float*>(slot0_ptr + scratch_off)[lane] = mine;
        float v[32];
#ifdef KB200_TRACE
        if (p.debug & 4) {
#pragma unroll
          for (int q = 0; q < 32; ++q) v[q] = 1.0f;
        } else
#endif
        tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * p.bn + c), v);
        __syncwarp();
#ifdef KB200_TRACE
        if (warp == 4 && lane == 0) { PAIR_STAMP(4, te); ++te; }
#endif
        run_chain(v, mine, n, batch);
        __syncwarp();
#ifdef KB200_TRACE
        if (warp == 4 && lane == 0) { PAIR_STAMP(4, te); ++te; }
#endif
        stage_rows(slot0_ptr, slot0_ptr + (with32 || has_res ? 4096 : 0), v, lane, with16, with32);
        fence_async_smem();
        __syncwarp();
#ifdef KB200_TRACE
        if (lane == 0 && !dry && !(p.debug & 1)) {
#else
        if (lane == 0 && !dry) {
#endif
          if (with32) tma_store_3d(&tma_out, slot0, n, m_first, batch);
          if (with16) tma_store_3d(&tma_out16, slot0 + (with32 || has_res ? 4096u : 0u), n, m_first, batch);
          tma_store_commit();
        }
#ifdef KB200_TRACE
        if (warp == 4 && lane == 0) { PAIR_STAMP(4, te); ++te; }
#endif
        if (dry) break;
      }
      if (dry) {
        dry = false;
        continue;
      }
      // this warp has read the accumulator: hand it back to the leader's MMA thread
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8 * acc);
      tile += num_pairs;
      ++i;
    }
    if (lane == 0) store_wait_read(0);   // shared memory must outlive the stores that read it
  }

  // ---------------- common exit ----------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
#ifdef KB200_TRACE
  if (blockIdx.x <= 1 && threadIdx.x == 0 && !(p.debug & 64)) {
    const long long t0 = marks[0];
    printf("PAIR block %d: alloc+sync done %lld cluster barrier done %lld after pdl %lld exit %lld | tiles %d bn %d stages %d num_kb %d grid %d\n",
           (int)blockIdx.x, marks[1] - t0, marks[2] - t0, marks[3] - t0, clock64() - t0, p.num_tiles, p.bn, p.stages, p.num_kb, (int)gridDim.x);
    for (int i2 = 0; i2 < 64; ++i2)
      printf("  b%d step %3d  prod_wait_done %7lld issued %7lld | mma_full %7lld committed %7lld\n", (int)blockIdx.x, i2, trace[0][i2] - t0,
             trace[1][i2] - t0, trace[2][i2] - t0, trace[3][i2] - t0);
    printf("  b%d epilogue warp 4 (tile ready; per block: loaded, slot free, computed, stored):", (int)blockIdx.x);
    for (int i2 = 0; i2 < 80; ++i2) printf(" %lld", trace[4][i2] - t0);
    printf("\n");
  }
#endif
  if (abort_flag && threadIdx.x == 0) {
    // copies may still be in flight towards this CTA's shared memory: give them a bounded time to land
    const long long t0 = clock64();
    while (clock64() - t0 < 400000) { }
  }
  // neither CTA leaves (or frees TMEM the other's MMAs write) before both are done
  cluster_arrive();
  cluster_wait();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)p.tmem_cols) : "memory");
  }
}

struct PairState {
  CUtensorMap map_a, map_b, map_out, map_out16, map_res;
  PairParams params;
  size_t smem_bytes = 0;
  dim3 grid;
  bool bf16 = false;
  void (*kernel)(CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, CUtensorMap, PairParams) = nullptr;
};

// The chain step operands the epilogue can take: immediates, unary ops, per-column vectors readable
// with 128-bit loads, and at most one full matrix that a bulk tensor load can describe.
bool classify_steps(const PlanKernel& k, PairParams* p, const DevOperand** res_operand) {
  int n_res = 0;
  if (p) { p->res_step = -1; p->n_steps = k.chain.n; }
  for (int s = 0; s < k.chain.n; ++s) {
    const ChainStep& cs = k.chain.steps[s];
    PairStep ps{};
    ps.op = cs.op;
    ps.imm = cs.imm;
    if (cs.slot == -1) {
      ps.kind = SIDE_IMM;
    } else if (cs.slot < 0) {
      ps.kind = SIDE_NONE;
    } else {
      const DevOperand& o = k.ops[cs.slot];
      if (o.stride[1] == 0 && o.stride[2] == 1 && o.stride[0] % 4 == 0 && aligned16(o.ptr)) {
        ps.kind = SIDE_COL;
        ps.ptr = o.ptr;
        ps.batch_stride = o.stride[0];
      } else if (o.stride[2] == 1 && o.stride[1] >= k.N && o.stride[1] % 4 == 0 && o.stride[0] % 4 == 0 && o.stride[0] >= 0 &&
                 aligned16(o.ptr) && ++n_res == 1) {
        ps.kind = SIDE_RES;
        if (p) { p->res_step = s; p->res_batched = (k.batch > 1 && o.stride[0] != 0) ? 1 : 0; }
        if (res_operand) *res_operand = &o;
      } else {
        return false;
      }
    }
    if (p) p->steps[s] = ps;
  }
  return true;
}

}  // namespace

bool pair_eligible(const Plan& plan, const PlanKernel& k) {
  const kb200_kernel_desc& d = k.desc;
  if (d.precision == KB200_PREC_FP32 || !k.has_chain) return false;
  if (d.cfg[0] == 128) return false;                       // the tuner asked for single-CTA tiles
  if (k.M <= 128 && d.cfg[0] != 256) return false;
  if (plan.sm_count < 2) return false;
  const bool bf16 = d.precision == KB200_PREC_BF16;
  const int chunk_n = bf16 ? 64 : 32;
  const DevOperand& B = k.ops[d.b_slot];
  const bool b_nmajor = B.stride[2] == 1;
  if (k.N < 128 || (b_nmajor && k.N % chunk_n)) return false;
  if (d.cfg[4] > 1) return false;                          // a forced split-K runs on the single-CTA kernel
  if (d.cfg[7] == 1 || d.cfg[7] == 2) return false;        // so do its epilogue variants
  if (((k.M + 255) / 256) * ((k.N + 127) / 128) * k.batch >= (int64_t(1) << 20)) return false;
  // bulk tensor stores: column-contiguous output, 16-byte aligned base and strides
  const DevOperand& O = k.ops[k.chain.out_slot];
  if (O.stride[2] != 1 || O.stride[1] % 4 || O.stride[1] < k.N || !aligned16(O.ptr)) return false;
  if (k.batch > 1 && (O.stride[0] % 4 || O.stride[0] <= 0)) return false;
  return classify_steps(k, nullptr, nullptr);
}

int pair_bind(Plan& plan, PlanKernel& k, int kernel_index, const PairOperands& ops, void** state) {
  const kb200_kernel_desc& d = k.desc;
  *state = nullptr;
  const DevOperand& O = k.ops[k.chain.out_slot];
  __nv_bfloat16* out16 = static_cast<__nv_bfloat16*>(k.shadow_out);
  if (out16 != nullptr && (O.stride[1] % 8 || (k.batch > 1 && O.stride[0] % 8) || !aligned16(out16))) return KB200_OK;
  PairState* st = new PairState();
  PairParams& p = st->params;
  const DevOperand* res = nullptr;
  if (!classify_steps(k, &p, &res)) { delete st; return KB200_OK; }
  st->bf16 = ops.bf16;
  if (ops.bf16)
    for (int s = 0; s < p.n_steps; ++s) {
      if (p.steps[s].op == CH_TANH) p.steps[s].op = CH_TANH_APPROX;
      else if (p.steps[s].op == CH_GELU_TANH) p.steps[s].op = CH_GELU_TANH_APPROX;
    }
  const int pairs = plan.sm_count / 2;
  const int slab_k = ops.bf16 ? 64 : 32, chunk_n = ops.bf16 ? 64 : 32;
  // Tile width and K slabs per pipeline step, by a cost model in cycles of the slowest SM pair.  A step
  // costs the issuing thread ~60 cycles per MMA plus ~250 for the probe and the commit, whatever the
  // width, and the tensor cores 2 cycles per column and slab: 256 columns are bound by the tensor
  // cores (512 per slab), 128 columns by the issue (~490, or ~365 with two slabs per step).  The
  // last tile's epilogue (~1200 cycles per 32-column block and warp) is not hidden.  When several
  // plans share the GPU (plan option CONCURRENCY) each can count on its share of the pairs only.
  int bn = d.cfg[1] == 128 || d.cfg[1] == 256 ? d.cfg[1] : 0;
  int kps = d.cfg[2] == 1 || d.cfg[2] == 2 ? d.cfg[2] : 0;
  const int share = plan.concurrency > 1 ? (pairs / plan.concurrency > 0 ? pairs / plan.concurrency : 1) : pairs;
  const int64_t slabs = (k.K + slab_k - 1) / slab_k;
  if (bn == 0) {
    int64_t best = 0;
    for (int cand : {256, 128}) {
      if (cand > 128 && cand / 2 >= k.N) continue;
      const int64_t n_tiles = ((k.M + 255) / 256) * ((k.N + cand - 1) / cand) * k.batch;
      const int64_t rounds = (n_tiles + share - 1) / share;
      const int64_t per_slab = cand == 256 ? 512 : (kps == 1 ? 490 : 365);
      const int64_t cost = rounds * slabs * per_slab + (cand / 64) * 1200;
      if (bn == 0 || cost < best) { bn = cand; best = cost; }
    }
  }
  while (bn > 128 && bn / 2 >= k.N) bn /= 2;
  // Staging per epilogue warp: one slot for a 32 x 32 block, float32 (also where a matrix operand of
  // the chain lands; left out when only the mirror is stored) and its bf16 copy.
  const bool store32 = !(k.mirror_only && out16 != nullptr);
  const int slot_bytes_wanted = ((store32 || p.res_step >= 0) ? 4096 : 0) + (out16 ? 2048 : 0);
  // two slabs per step where the ring still has three stages beside the staging slots
  if (kps == 0)
    kps = bn <= 128 && slabs >= 4 && 3 * 2 * (kPairATileBytes + bn / 2 * 128) + kPairEpiWarps * slot_bytes_wanted + 1024 <= kPairSmemCeiling ? 2 : 1;
  p.bn = bn;
  p.half_bn = bn / 2;
  p.slab_k = slab_k;
  p.kps = kps;
  p.step_k = kps * slab_k;
  p.num_kb = (int)((k.K + p.step_k - 1) / p.step_k);
  p.b_kmajor = ops.b_kmajor ? 1 : 0;
  p.chunk_n = chunk_n;
  p.b_lbo_bytes = (uint32_t)(p.step_k * 128);              // N-major: bytes between the column chunks of a stage
  p.b_sbo_bytes = ops.bf16 ? 1024 : 512;
  // An N-major operand of 32-bit elements uses the 128-byte swizzle on 32-byte atoms (pattern of 4 rows);
  // 16-bit elements the ordinary 128-byte swizzle (8 rows).
  p.b_layout = ops.bf16 ? 2 : 1;
  p.b_step16 = ops.b_kmajor ? 2u : (uint32_t)((ops.bf16 ? 16 : 8) * 128) >> 4;
  p.b_slab16 = ops.b_kmajor ? (uint32_t)(p.half_bn * 128) >> 4 : 4u * p.b_step16;
  const uint32_t fmt = ops.bf16 ? 1u : 2u;
  // instruction descriptor: D = F32, A/B = BF16 or TF32, A K-major, B as bound, N = bn, M = 256 over the pair
  p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((ops.b_kmajor ? 0u : 1u) << 16) | ((uint32_t)(bn >> 3) << 17) | ((256u >> 4) << 24);
  p.tmem_cols = 32;
  while (p.tmem_cols < 2 * bn) p.tmem_cols *= 2;
  p.tiles_n = (int)((k.N + bn - 1) / bn);
  const int tiles_m = (int)((k.M + 255) / 256);
  p.tiles_per_batch = tiles_m * p.tiles_n;
  p.num_tiles = p.tiles_per_batch * (int)k.batch;
  p.magic_tn = ((uint64_t(1) << 40) + p.tiles_n - 1) / p.tiles_n;
  p.magic_tpb = ((uint64_t(1) << 40) + p.tiles_per_batch - 1) / p.tiles_per_batch;
  p.kernel_index = kernel_index;
  p.status = plan.d_status;
#ifdef KB200_TRACE
  p.debug = getenv("KB200_PAIR_DEBUG") ? atoi(getenv("KB200_PAIR_DEBUG")) : 0;
#endif
  p.M = k.M;
  p.N = k.N;
  p.out16 = out16;
  p.store32 = store32 ? 1 : 0;
  p.slot_bytes = slot_bytes_wanted;
  p.slots = 1;
  const int stage_bytes = kps * (kPairATileBytes + p.half_bn * 128);
  const int epi_bytes = kPairEpiWarps * p.slot_bytes;
  int stages = d.cfg[3] > 0 ? d.cfg[3] : kPairMaxStages;
  if (stages > kPairMaxStages) stages = kPairMaxStages;
  while (stages > 2 && (size_t)stages * stage_bytes + epi_bytes + 1024 > (size_t)kPairSmemCeiling) --stages;
  if ((size_t)stages * stage_bytes + epi_bytes + 1024 > (size_t)kPairSmemCeiling) { delete st; return KB200_OK; }
  p.stages = stages;
  st->smem_bytes = (size_t)stages * stage_bytes + epi_bytes + 1024;
  // Persistent pairs: as many as there are tiles, up to this plan's share of the GPU.  With several
  // plans in flight a kernel that spread one tile to every pair would leave each pair's tensor cores
  // idle through its epilogue (bound by the store path, longer than the main loop at K = 768); on its
  // share of the pairs every pair walks several tiles and drains one while it multiplies the next.
  const int rounds = (p.num_tiles + share - 1) / share;
  const int n_pairs = (p.num_tiles + rounds - 1) / rounds;
  st->grid = dim3((unsigned)(2 * n_pairs), 1, 1);

  bool ok = encode_map(&st->map_a, ops.bf16, ops.a_base, k.K, k.M, k.batch, ops.a_row, ops.a_batch, slab_k, 128, false);
  if (ok) {
    if (ops.b_kmajor)
      ok = encode_map(&st->map_b, ops.bf16, ops.b_base, k.K, k.N, k.batch, ops.b_row, ops.b_batch, slab_k, p.half_bn, false);
    else
      ok = encode_map4(&st->map_b, ops.bf16, ops.b_base, chunk_n, k.K, k.N / chunk_n, k.batch, ops.b_row, ops.b_batch, p.step_k,
                       p.half_bn / chunk_n, !ops.bf16);
  }
  if (ok) ok = encode_map_store(&st->map_out, false, O.ptr, k.N, k.M, k.batch, O.stride[1], O.stride[0]);
  st->map_out16 = st->map_out;
  st->map_res = st->map_out;
  if (ok && out16) ok = encode_map_store(&st->map_out16, true, out16, k.N, k.M, k.batch, O.stride[1], O.stride[0]);
  if (ok && res) ok = encode_map_store(&st->map_res, false, res->ptr, k.N, k.M, p.res_batched ? k.batch : 1, res->stride[1], res->stride[0]);
  if (!ok) { delete st; return KB200_OK; }
  st->kernel = ops.bf16 ? (kps == 2 ? mm_pair_kernel<true, 2> : mm_pair_kernel<true, 1>)
                        : (kps == 2 ? mm_pair_kernel<false, 2> : mm_pair_kernel<false, 1>);
  cudaError_t e = cudaFuncSetAttribute(st->kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemCeiling);
  if (e != cudaSuccess) { delete st; return cuda_fail(e, "cudaFuncSetAttribute(mm_pair_kernel)"); }
  *state = st;
  return KB200_OK;
}

int pair_launch(const Plan& plan, const void* state, cudaStream_t s) {
  const PairState* st = static_cast<const PairState*>(state);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = st->grid;
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = st->smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  int n_attr = 0;
  attr[n_attr].id = cudaLaunchAttributeClusterDimension;
  attr[n_attr].val.clusterDim.x = 2;
  attr[n_attr].val.clusterDim.y = 1;
  attr[n_attr].val.clusterDim.z = 1;
  ++n_attr;
  if (plan.pdl) {
    attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
    ++n_attr;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n_attr;
  KB200_CUDA(cudaLaunchKernelEx(&cfg, st->kernel, st->map_a, st->map_b, st->map_out, st->map_out16, st->map_res, st->params));
  KB200_CUDA(cudaGetLastError());
  return KB200_OK;
}

void pair_destroy(void* state) { delete static_cast<PairState*>(state); }

}  // namespace kb200
