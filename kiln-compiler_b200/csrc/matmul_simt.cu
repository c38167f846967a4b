// Exact-FP32 batched matmul with a fused epilogue, on the FP32 pipes.  Role of the reference's
// matmul generator with input_precision="ieee" (kiln/gpu/codegen.py:484-530): arbitrary strided
// A [batch, M, K] and B [batch, K, N], FP32 accumulation over K, the epilogue applied to the
// accumulator while it is still in registers, out-of-range tile elements read as 0 and are not
// stored (codegen.py:513-517, 524).  tcgen05 has no IEEE-FP32 operand kind, so this is the path
// for allow_tf32=False; it is also the fallback for operands the tensor-core path cannot take.
#include "device_math.cuh"
#include "kb200_internal.h"
#include "matmul.h"

namespace kb200 {

template <int BM, int BN, int BK, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN)) mm_simt_kernel(const __grid_constant__ MatmulParams p) {
  pdl_wait();                 // the producer of this kernel's inputs has completed
  pdl_launch_dependents();    // the next kernel may begin its start-up
  constexpr int NT = (BM / TM) * (BN / TN);
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN), ty = tid / (BN / TN);
  const int64_t tiles_n = (p.N + BN - 1) / BN;
  const int64_t m0 = (blockIdx.x / tiles_n) * BM, n0 = (blockIdx.x % tiles_n) * BN;
  const int64_t b = blockIdx.z;
  const float* A = p.ops[p.a_slot].ptr + b * p.ops[p.a_slot].stride[0];
  const float* B = p.ops[p.b_slot].ptr + b * p.ops[p.b_slot].stride[0];
  const int64_t a_sm = p.ops[p.a_slot].stride[1], a_sk = p.ops[p.a_slot].stride[2];
  const int64_t b_sk = p.ops[p.b_slot].stride[1], b_sn = p.ops[p.b_slot].stride[2];
  const bool a_kfast = a_sk == 1 || a_sm != 1;
  const bool b_nfast = b_sn == 1 || b_sk != 1;

  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

  for (int64_t k0 = 0; k0 < p.K; k0 += BK) {
#pragma unroll
    for (int e = tid; e < BM * BK; e += NT) {
      const int kk = a_kfast ? e % BK : e / BM;
      const int mm = a_kfast ? e / BK : e % BM;
      const int64_t gm = m0 + mm, gk = k0 + kk;
      As[kk][mm] = (gm < p.M && gk < p.K) ? A[gm * a_sm + gk * a_sk] : 0.0f;
    }
#pragma unroll
    for (int e = tid; e < BK * BN; e += NT) {
      const int nn = b_nfast ? e % BN : e / BK;
      const int kk = b_nfast ? e / BN : e % BK;
      const int64_t gn = n0 + nn, gk = k0 + kk;
      Bs[kk][nn] = (gn < p.N && gk < p.K) ? B[gk * b_sk + gn * b_sn] : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], bb[TN];
#pragma unroll
      for (int i = 0; i < TM; i += 4) {
        const float4 t = *reinterpret_cast<const float4*>(&As[kk][ty * TM + i]);
        a[i] = t.x; a[i + 1] = t.y; a[i + 2] = t.z; a[i + 3] = t.w;
      }
#pragma unroll
      for (int j = 0; j < TN; j += 4) {
        const float4 t = *reinterpret_cast<const float4*>(&Bs[kk][tx * TN + j]);
        bb[j] = t.x; bb[j + 1] = t.y; bb[j + 2] = t.z; bb[j + 3] = t.w;
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], bb[j], acc[i][j]);
    }
    __syncthreads();
  }

  // ---- epilogue ----
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int64_t gm = m0 + ty * TM + i;
    if (gm >= p.M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int64_t gn = n0 + tx * TN + j;
      if (gn >= p.N) continue;
      epilogue_store(p, acc[i][j], b, gm, gn);
    }
  }
}

// Decode shape, M == 1: the weight matrix is read exactly once, so the kernel is bound by how many
// bytes it keeps in flight.  Each CTA owns 32 output columns (one per lane: a warp reads 128
// contiguous bytes of a row of B); its 32 warps split K, each with up to sixteen rows in flight (6 MB
// over the 96 CTAs of a 3072-wide layer), and combine through shared memory in warp order, which
// keeps the result deterministic.  (64 columns and 8 warps with four rows in flight gave 48 CTAs and
// 0.9 TB/s; staging the vector in shared memory to have 32 rows in flight measured slower.)
constexpr int kGemvWarps = 32;
constexpr int kGemvCols = 32;
__global__ void __launch_bounds__(kGemvWarps * 32) mm_gemv_kernel(const __grid_constant__ MatmulParams p) {
  pdl_wait();                 // the producer of this kernel's inputs has completed
  pdl_launch_dependents();    // the next kernel may begin its start-up
  __shared__ float part[kGemvWarps][kGemvCols];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t b = blockIdx.z;
  const float* A = p.ops[p.a_slot].ptr + b * p.ops[p.a_slot].stride[0];
  const float* B = p.ops[p.b_slot].ptr + b * p.ops[p.b_slot].stride[0];
  const int64_t a_sk = p.ops[p.a_slot].stride[2];
  const int64_t b_sk = p.ops[p.b_slot].stride[1];
  const int64_t n = (int64_t)blockIdx.x * kGemvCols + lane;
  const int64_t k_per = (p.K + kGemvWarps - 1) / kGemvWarps;
  const int64_t k_lo = warp * k_per, k_hi = (k_lo + k_per < p.K) ? k_lo + k_per : p.K;
  float acc = 0.0f;
  if (n < p.N) {
    int64_t k = k_lo;
    for (; k + 16 <= k_hi; k += 16) {
      float w[16], a[16];
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        w[u] = __ldg(B + (k + u) * b_sk + n);
        a[u] = __ldg(A + (k + u) * a_sk);
      }
#pragma unroll
      for (int u = 0; u < 16; ++u) acc = fmaf(a[u], w[u], acc);
    }
    for (; k + 8 <= k_hi; k += 8) {
      float w[8], a[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        w[u] = __ldg(B + (k + u) * b_sk + n);
        a[u] = __ldg(A + (k + u) * a_sk);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) acc = fmaf(a[u], w[u], acc);
    }
    for (; k < k_hi; ++k) acc = fmaf(__ldg(A + k * a_sk), __ldg(B + k * b_sk + n), acc);
  }
  part[warp][lane] = acc;
  __syncthreads();
  if (threadIdx.x < kGemvCols) {
    const int64_t gn = (int64_t)blockIdx.x * kGemvCols + threadIdx.x;
    if (gn < p.N) {
      float t = 0.0f;
#pragma unroll
      for (int w = 0; w < kGemvWarps; ++w) t += part[w][threadIdx.x];
      epilogue_store(p, t, b, 0, gn);
    }
  }
}

void fill_matmul_params(const PlanKernel& k, MatmulParams* p) {
  const kb200_kernel_desc& d = k.desc;
  p->batch = k.batch;
  p->M = k.M;
  p->N = k.N;
  p->K = k.K;
  p->a_slot = d.a_slot;
  p->b_slot = d.b_slot;
  p->n_operands = k.n_ops;
  for (int o = 0; o < k.n_ops; ++o) p->ops[o] = k.ops[o];
  p->has_chain = k.has_chain ? 1 : 0;
  p->chain = k.chain;
  p->tape = k.tape;
}

int launch_matmul_simt(const Plan& plan, const PlanKernel& k, cudaStream_t s) {
  MatmulParams p{};
  fill_matmul_params(k, &p);
  if (k.impl == IMPL_MM_GEMV) {
    dim3 grid((unsigned)((p.N + kGemvCols - 1) / kGemvCols), 1, (unsigned)p.batch);
    launch_kernel(plan.pdl, mm_gemv_kernel, grid, dim3(kGemvWarps * 32), 0, s, p);
  } else {
    const int64_t big_tiles = ((p.M + 127) / 128) * ((p.N + 127) / 128) * p.batch;
    if (big_tiles >= plan.sm_count) {
      dim3 grid((unsigned)(((p.M + 127) / 128) * ((p.N + 127) / 128)), 1, (unsigned)p.batch);
      launch_kernel(plan.pdl, mm_simt_kernel<128, 128, 8, 8, 8>, grid, dim3(256), 0, s, p);
    } else {
      dim3 grid((unsigned)(((p.M + 63) / 64) * ((p.N + 63) / 64)), 1, (unsigned)p.batch);
      launch_kernel(plan.pdl, mm_simt_kernel<64, 64, 16, 4, 4>, grid, dim3(256), 0, s, p);
    }
  }
  KB200_CUDA(cudaGetLastError());
  return KB200_OK;
}

}  // namespace kb200
