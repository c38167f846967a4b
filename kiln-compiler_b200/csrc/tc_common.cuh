// Pieces shared by the tcgen05 kernels (matmul, attention): mbarrier / TMA / tcgen05 wrappers in
// inline PTX, shared-memory matrix descriptors, and the host-side TMA tensor-map encoder.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kb200 {
namespace tc {

constexpr uint32_t kWaitLimit = 1u << 20;   // polls of an mbarrier before a wait gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Two float32 operations per instruction (sm_100 packed forms) and the three-input maximum: the
// softmax warps and the matmul epilogues are bound by instruction issue, not by the FP32 pipes.
__device__ __forceinline__ float2 ffma2(float2 a, float2 b, float2 c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)),
        "l"(*reinterpret_cast<unsigned long long*>(&c)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fadd2(float2 a, float2 b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float2 fmul2(float2 a, float2 b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;"
      : "=l"(d)
      : "l"(*reinterpret_cast<unsigned long long*>(&a)), "l"(*reinterpret_cast<unsigned long long*>(&b)));
  return *reinterpret_cast<float2*>(&d);
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false if the limit ran out or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63) == 63 && *abort_flag) return false;
  }
  return false;
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Bulk tensor store shared -> global of one box (bulk async-group completion).  The part of the box
// that lies outside the tensor is not written.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// All earlier store groups of this thread have finished READING shared memory (it may be rewritten).
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// All but the two most recent store groups of this thread have finished reading shared memory.
__device__ __forceinline__ void tma_store_wait_read2() { asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory"); }
// Makes this thread's shared-memory writes visible to the async proxy (TMA) before a store is issued.
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout = 2) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version for sm_100
  d |= (uint64_t)layout << 61;
  return d;
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                     bool bf16) {
  if (bf16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Two 32-column loads in flight at once, one wait: the latency of a tensor-memory load is what an
// epilogue warp waits for, not its bandwidth.
__device__ __forceinline__ void tmem_ld32x2(uint32_t taddr_a, uint32_t taddr_b, float (&va)[32], float (&vb)[32]) {
  uint32_t ra[32], rb[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(ra[0]), "=r"(ra[1]), "=r"(ra[2]), "=r"(ra[3]), "=r"(ra[4]), "=r"(ra[5]), "=r"(ra[6]), "=r"(ra[7]), "=r"(ra[8]), "=r"(ra[9]), "=r"(ra[10]), "=r"(ra[11]), "=r"(ra[12]), "=r"(ra[13]), "=r"(ra[14]), "=r"(ra[15]), "=r"(ra[16]), "=r"(ra[17]), "=r"(ra[18]), "=r"(ra[19]), "=r"(ra[20]), "=r"(ra[21]), "=r"(ra[22]), "=r"(ra[23]), "=r"(ra[24]), "=r"(ra[25]), "=r"(ra[26]), "=r"(ra[27]), "=r"(ra[28]), "=r"(ra[29]), "=r"(ra[30]), "=r"(ra[31]),
        "=r"(rb[0]), "=r"(rb[1]), "=r"(rb[2]), "=r"(rb[3]), "=r"(rb[4]), "=r"(rb[5]), "=r"(rb[6]), "=r"(rb[7]), "=r"(rb[8]), "=r"(rb[9]), "=r"(rb[10]), "=r"(rb[11]), "=r"(rb[12]), "=r"(rb[13]), "=r"(rb[14]), "=r"(rb[15]), "=r"(rb[16]), "=r"(rb[17]), "=r"(rb[18]), "=r"(rb[19]), "=r"(rb[20]), "=r"(rb[21]), "=r"(rb[22]), "=r"(rb[23]), "=r"(rb[24]), "=r"(rb[25]), "=r"(rb[26]), "=r"(rb[27]), "=r"(rb[28]), "=r"(rb[29]), "=r"(rb[30]), "=r"(rb[31])
      : "r"(taddr_a), "r"(taddr_b)
      : "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) { va[i] = __uint_as_float(ra[i]); vb[i] = __uint_as_float(rb[i]); }
}

// The same two loads without the wait, and the wait as a statement of its own that names the
// registers as in-out operands (nothing that reads them may be scheduled above it): other work --
// a tensor-memory store, a barrier arrival -- goes between the two.
__device__ __forceinline__ void tmem_ld32x2_issue(uint32_t taddr_a, uint32_t taddr_b, uint32_t (&ra)[32], uint32_t (&rb)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];"
      : "=r"(ra[0]), "=r"(ra[1]), "=r"(ra[2]), "=r"(ra[3]), "=r"(ra[4]), "=r"(ra[5]), "=r"(ra[6]), "=r"(ra[7]), "=r"(ra[8]), "=r"(ra[9]), "=r"(ra[10]), "=r"(ra[11]), "=r"(ra[12]), "=r"(ra[13]), "=r"(ra[14]), "=r"(ra[15]), "=r"(ra[16]), "=r"(ra[17]), "=r"(ra[18]), "=r"(ra[19]), "=r"(ra[20]), "=r"(ra[21]), "=r"(ra[22]), "=r"(ra[23]), "=r"(ra[24]), "=r"(ra[25]), "=r"(ra[26]), "=r"(ra[27]), "=r"(ra[28]), "=r"(ra[29]), "=r"(ra[30]), "=r"(ra[31]), "=r"(rb[0]), "=r"(rb[1]), "=r"(rb[2]), "=r"(rb[3]), "=r"(rb[4]), "=r"(rb[5]), "=r"(rb[6]), "=r"(rb[7]), "=r"(rb[8]), "=r"(rb[9]), "=r"(rb[10]), "=r"(rb[11]), "=r"(rb[12]), "=r"(rb[13]), "=r"(rb[14]), "=r"(rb[15]), "=r"(rb[16]), "=r"(rb[17]), "=r"(rb[18]), "=r"(rb[19]), "=r"(rb[20]), "=r"(rb[21]), "=r"(rb[22]), "=r"(rb[23]), "=r"(rb[24]), "=r"(rb[25]), "=r"(rb[26]), "=r"(rb[27]), "=r"(rb[28]), "=r"(rb[29]), "=r"(rb[30]), "=r"(rb[31])
      : "r"(taddr_a), "r"(taddr_b)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait64(uint32_t (&ra)[32], uint32_t (&rb)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(ra[0]), "+r"(ra[1]), "+r"(ra[2]), "+r"(ra[3]), "+r"(ra[4]), "+r"(ra[5]), "+r"(ra[6]), "+r"(ra[7]), "+r"(ra[8]), "+r"(ra[9]), "+r"(ra[10]), "+r"(ra[11]), "+r"(ra[12]), "+r"(ra[13]), "+r"(ra[14]), "+r"(ra[15]), "+r"(ra[16]), "+r"(ra[17]), "+r"(ra[18]), "+r"(ra[19]), "+r"(ra[20]), "+r"(ra[21]), "+r"(ra[22]), "+r"(ra[23]), "+r"(ra[24]), "+r"(ra[25]), "+r"(ra[26]), "+r"(ra[27]), "+r"(ra[28]), "+r"(ra[29]), "+r"(ra[30]), "+r"(ra[31]), "+r"(rb[0]), "+r"(rb[1]), "+r"(rb[2]), "+r"(rb[3]), "+r"(rb[4]), "+r"(rb[5]), "+r"(rb[6]), "+r"(rb[7]), "+r"(rb[8]), "+r"(rb[9]), "+r"(rb[10]), "+r"(rb[11]), "+r"(rb[12]), "+r"(rb[13]), "+r"(rb[14]), "+r"(rb[15]), "+r"(rb[16]), "+r"(rb[17]), "+r"(rb[18]), "+r"(rb[19]), "+r"(rb[20]), "+r"(rb[21]), "+r"(rb[22]), "+r"(rb[23]), "+r"(rb[24]), "+r"(rb[25]), "+r"(rb[26]), "+r"(rb[27]), "+r"(rb[28]), "+r"(rb[29]), "+r"(rb[30]), "+r"(rb[31])
               :
               : "memory");
}

// tcgen05.mma with the A operand read from tensor memory (M x K, one 32-bit element per column)
// and B from shared memory.
__device__ __forceinline__ void umma_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                        bool bf16) {
  if (bf16) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])),
        "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])),
        "r"(__float_as_uint(v[11])), "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])),
        "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])),
        "r"(__float_as_uint(v[23])), "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])),
        "r"(__float_as_uint(v[31]))
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// ---- thread-block clusters ----
// The two halves of the hardware cluster barrier, usable apart: arrive early, wait when the result is needed.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// Arrive on an mbarrier of another CTA of the cluster (address from map_to_cta); orders this thread's
// earlier writes -- and, through a preceding CTA barrier, its CTA's -- before the arrival, cluster-wide.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t remote_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote_bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((i & 63) == 63 && *abort_flag) return false;
  }
  return false;
}
// The same for a wait that is expected to last (an epilogue warp waiting for its tile): the thread
// sleeps between polls, so that sixteen waiting warps leave the issue slots and the barrier's
// shared-memory bank to the threads that feed the tensor cores.
__device__ __forceinline__ bool mbar_wait_cluster_relaxed(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    __nanosleep(100);
    if ((i & 63) == 63 && *abort_flag) return false;
  }
  return false;
}
// Shared-memory address of the same location in the CTA with rank `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
  return remote;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}

// ---- host side ----
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  }
  return fn;
}

// A 3-D tiled map over [batch, rows, cols] with cols contiguous; box = (box_cols, box_rows, 1).
inline bool encode_map(CUtensorMap* map, bool bf16, const void* base, int64_t cols, int64_t rows, int64_t batch,
                int64_t row_stride_elems, int64_t batch_stride_elems, int box_cols, int box_rows, bool atom32) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const int esz = bf16 ? 2 : 4;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)row_stride_elems * esz, (cuuint64_t)(batch > 1 ? batch_stride_elems : row_stride_elems * rows) * esz};
  if (strides[1] == 0) strides[1] = strides[0] * rows;
  cuuint32_t box[3] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows, 1};
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base),
                  dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// A 4-D tiled map over an N-major matrix [batch, rows, n_chunks * chunk] seen as
// (chunk, rows, n_chunks, batch): one box (chunk, box_rows, box_chunks, 1) lands in shared memory as
// box_chunks consecutive blocks of [box_rows x chunk], the layout the N-major MMA descriptor walks.
inline bool encode_map4(CUtensorMap* map, bool bf16, const void* base, int chunk, int64_t rows, int64_t n_chunks, int64_t batch,
                        int64_t row_stride_elems, int64_t batch_stride_elems, int box_rows, int box_chunks, bool atom32) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const int esz = bf16 ? 2 : 4;
  cuuint64_t dims[4] = {(cuuint64_t)chunk, (cuuint64_t)rows, (cuuint64_t)n_chunks, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)row_stride_elems * esz, (cuuint64_t)chunk * esz,
                           (cuuint64_t)(batch > 1 ? batch_stride_elems : row_stride_elems * rows) * esz};
  if (strides[2] == 0) strides[2] = strides[0] * rows;
  cuuint32_t box[4] = {(cuuint32_t)chunk, (cuuint32_t)box_rows, (cuuint32_t)box_chunks, 1};
  cuuint32_t elem[4] = {1, 1, 1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(base),
                  dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  atom32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

// A 3-D map over [batch, rows, cols] (cols contiguous) for bulk stores of 32 x 32 blocks staged in
// shared memory with rows of 128 bytes (float, 128-byte swizzle) or 64 bytes (bf16, 64-byte swizzle):
// the swizzle lets both a lane-per-row and a lane-per-column writer fill the block without bank conflicts.
// Bulk-store map over [batch, rows, cols] with boxes of 32 rows x 128 bytes (32 floats; `wide`: 64 bf16)
// under the 128-byte swizzle, or 32 rows x 32 bf16 under the 64-byte swizzle.
inline bool encode_map_store(CUtensorMap* map, bool bf16, const void* base, int64_t cols, int64_t rows, int64_t batch,
                             int64_t row_stride_elems, int64_t batch_stride_elems, bool wide = false) {
  EncodeFn fn = encode_fn();
  if (!fn) return false;
  const int esz = bf16 ? 2 : 4;
  cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)row_stride_elems * esz, (cuuint64_t)(batch > 1 ? batch_stride_elems : row_stride_elems * rows) * esz};
  if (strides[1] == 0) strides[1] = strides[0] * rows;
  cuuint32_t box[3] = {bf16 && wide ? 64u : 32u, 32, 1};
  cuuint32_t elem[3] = {1, 1, 1};
  CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base),
                  dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  bf16 && !wide ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }


}  // namespace tc
}  // namespace kb200
