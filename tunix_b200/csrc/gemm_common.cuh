// Pieces shared by the 1-CTA and 2-CTA GEMM kernels: launch parameters, tile ordering and the
// epilogue that turns 32 fp32 accumulator columns of one row into global-memory stores.
#pragma once

#include "tx_ptx.cuh"

namespace txg {

struct GemmParams {
  void* C;
  long long ldc;
  int M, N, K;
  int c_fp32;      // 1: C is fp32, 0: C is bf16
  int accumulate;  // 1: C += result, 0: C = result
  float alpha;
  int* status;
  int k_splits;    // > 1: every tile is computed by k_splits CTAs over disjoint K ranges; C must then be a zeroed
                   // fp32 buffer and the epilogue adds into it atomically (single-CTA kernel only)
  int K2;          // > 0: a second operand pair (A2 [M,K2], B2 [N,K2], same layouts) is accumulated after the first:
                   // C = A B^T + A2 B2^T in one pass (fused low-rank adapters); 0 otherwise
  int n_red;       // > 0: all-reduce epilogue - the tile is added (fp32 vector atomics) into each of the n_red
  float* red_dst[8];   // zero-filled [M, N] buffers, one per rank of a tensor-parallel group (peer-mapped memory),
                       // so after every rank's GEMM each buffer holds the full sum (single-CTA kernel only)
};

// Walks tiles so that `group_m` consecutive row-blocks share their B tiles while they are hot in L2.
__device__ __forceinline__ void tile_coords(int t, int mb, int nb, int group_m, int& pm, int& pn) {
  const int per_group = group_m * nb;
  const int g = t / per_group;
  const int first_m = g * group_m;
  const int gsize = min(mb - first_m, group_m);
  const int r = t - g * per_group;
  pm = first_m + (r % gsize);
  pn = r / gsize;
}

// r[0..31]: accumulator columns [col, col + 32) of row `row`.
__device__ __forceinline__ void store_row_chunk(const GemmParams& p, int row, int col, const uint32_t (&r)[32]) {
  if (row >= p.M || col >= p.N) return;
  if (p.k_splits > 1 || p.n_red > 0) {
    const int nd = p.n_red > 0 ? p.n_red : 1;
    for (int d = 0; d < nd; ++d) {
      float* base = p.n_red > 0 ? p.red_dst[d] : reinterpret_cast<float*>(p.C);
      float* dst = base + static_cast<long long>(row) * p.ldc + col;
      if (p.n_red > 0) {
        // peer-mapped destinations: plain scalar fp32 atomics, which NVLink carries natively
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (col + j < p.N) atomicAdd(dst + j, __uint_as_float(r[j]) * p.alpha);
        continue;
      }
#pragma unroll
      for (int j = 0; j < 32; j += 4) {
        if (col + j < p.N)
          asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j),
                       "f"(__uint_as_float(r[j]) * p.alpha), "f"(__uint_as_float(r[j + 1]) * p.alpha),
                       "f"(__uint_as_float(r[j + 2]) * p.alpha), "f"(__uint_as_float(r[j + 3]) * p.alpha)
                       : "memory");
      }
    }
    return;
  }
  if (p.c_fp32) {
    float* dst = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      if (col + j < p.N) {
        float4 v = make_float4(__uint_as_float(r[j]) * p.alpha, __uint_as_float(r[j + 1]) * p.alpha,
                               __uint_as_float(r[j + 2]) * p.alpha, __uint_as_float(r[j + 3]) * p.alpha);
        float4* d4 = reinterpret_cast<float4*>(dst + j);
        if (p.accumulate) {
          const float4 o = *d4;
          v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
        }
        *d4 = v;
      }
    }
  } else {
    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col;
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      if (col + j < p.N) {
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[j + e]) * p.alpha;
        uint4* d4 = reinterpret_cast<uint4*>(dst + j);
        if (p.accumulate) {
          const uint4 o = *d4;
          const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 of = __bfloat1622float2(o2[e]);
            f[2 * e] += of.x;
            f[2 * e + 1] += of.y;
          }
        }
        uint4 v;
        __nv_bfloat162* v2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
        for (int e = 0; e < 4; ++e) v2[e] = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
        *d4 = v;
      }
    }
  }
}

}  // namespace txg

// Implemented in gemm_tcgen05_pair.cu: the 2-CTA (256 x 256 tile per CTA pair) variant.
int tx_gemm_pair_launch(const void* A, const void* B, const void* A2, const void* B2, const txg::GemmParams& p,
                        long long lda, long long ldb, long long lda2, long long ldb2, int a_mn, int b_mn, int max_ctas,
                        cudaStream_t stream);
