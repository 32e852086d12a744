// Expert-parallel token exchange for mixture-of-experts layers, written as kernels over
// peer-mapped (NVLink / NVSwitch) memory instead of an all-to-all collective.
//
//   tx_moe_dispatch_rows : every routed row (token, slot) is copied - optionally scaled - straight
//                          into its destination rank's receive buffer, at the row the routing plan
//                          gives it (expert-major, 128-row-padded layout of the grouped GEMM).
//   tx_moe_combine_rows  : every token pulls its k expert outputs from the owning ranks' result
//                          buffers, weights them and sums them in fp32; optionally keeps the k
//                          pulled rows (the backward of the weighting needs them).
// Both use plain 16-byte peer loads / stores. Ordering between ranks (buffer free / rows landed) is
// the caller's: a tx_peer_barrier before and after, on the same stream.
// A destination row outside the buffer (capacity overflow) is skipped and sets status bit 8.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tx_host.h"

namespace {

constexpr int kMaxPeers = 16;

struct PeerTable {
  void* p[kMaxPeers];
};

__device__ __forceinline__ uint4 scale8(uint4 v, float s) {
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float2 f = __bfloat1622float2(h[e]);
    h[e] = __floats2bfloat162_rn(f.x * s, f.y * s);
  }
  return v;
}

// One warp per routed row. src row = tok[i] (or i / k when tok is null).
__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const __nv_bfloat16* __restrict__ src, long long ld, const int* __restrict__ tok, int k,
                    const float* __restrict__ scale, const int* __restrict__ dest_rank,
                    const int* __restrict__ dest_row, PeerTable recv, int world, long long n, int D,
                    long long capacity, int* status) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const long long nwarps = (gridDim.x * static_cast<long long>(blockDim.x)) >> 5;
  const int d8 = D / 8;
  for (long long i = warp0; i < n; i += nwarps) {
    const int dr = __ldg(dest_rank + i);
    const long long row = __ldg(dest_row + i);
    if (dr < 0 || dr >= world || row < 0 || row >= capacity) {
      if (lane == 0) atomicOr(status, 8);
      continue;
    }
    const long long t = tok ? __ldg(tok + i) : i / k;
    const uint4* s = reinterpret_cast<const uint4*>(src + t * ld);
    uint4* d = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(recv.p[dr]) + row * D);
    if (scale) {
      const float w = __ldg(scale + i);
      for (int c = lane; c < d8; c += 32) d[c] = scale8(__ldg(s + c), w);
    } else {
      for (int c = lane; c < d8; c += 32) d[c] = __ldg(s + c);
    }
  }
}

// One CTA of 128 threads per token; thread c handles 16-byte chunks c, c + 128, ...
template <int KMAX>
__global__ void __launch_bounds__(128)
moe_combine_kernel(PeerTable send, int world, const int* __restrict__ dest_rank, const int* __restrict__ dest_row,
                   const float* __restrict__ weights, int k, __nv_bfloat16* __restrict__ out, long long ldo,
                   __nv_bfloat16* __restrict__ gathered, long long T, int D, long long capacity, int* status) {
  const int d8 = D / 8;
  for (long long t = blockIdx.x; t < T; t += gridDim.x) {
    const uint4* rows[KMAX];
    float w[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) {
      rows[j] = nullptr;
      w[j] = 0.f;
      if (j < k) {
        const int dr = __ldg(dest_rank + t * k + j);
        const long long row = __ldg(dest_row + t * k + j);
        if (dr < 0 || dr >= world || row < 0 || row >= capacity) {
          if (threadIdx.x == 0) atomicOr(status, 8);
        } else {
          rows[j] = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(send.p[dr]) + row * D);
          w[j] = weights ? __ldg(weights + t * k + j) : 1.f;
        }
      }
    }
    for (int c = threadIdx.x; c < d8; c += blockDim.x) {
      uint4 v[KMAX];
#pragma unroll
      for (int j = 0; j < KMAX; ++j)          // all k peer loads are in flight before the first use
        v[j] = (j < k && rows[j]) ? rows[j][c] : make_uint4(0, 0, 0, 0);
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int j = 0; j < KMAX; ++j) {
        if (j < k) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v[j]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(h[e]);
            acc[2 * e] += w[j] * f.x;
            acc[2 * e + 1] += w[j] * f.y;
          }
          if (gathered) reinterpret_cast<uint4*>(gathered + (t * k + j) * D)[c] = v[j];
        }
      }
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[2 * e], acc[2 * e + 1]);
      reinterpret_cast<uint4*>(out + t * ldo)[c] = o;
    }
  }
}

}  // namespace

// src [T, D] bf16 (row stride ld); routed row i reads token tok[i] (tok == null: token i / k) and lands in
// recv_ptrs[dest_rank[i]] at row dest_row[i] of a [capacity, D] bf16 buffer. scale (fp32 [n]) may be null.
extern "C" int tx_moe_dispatch_rows(const void* src, long long ld, const int* tok, int k, const float* scale,
                                    const int* dest_rank, const int* dest_row, void* const* recv_ptrs, int world,
                                    long long n, int D, long long capacity, int* status, cudaStream_t s) {
  if (world < 1 || world > kMaxPeers || (D & 7) || (ld & 7) || k < 1) return 1;
  if (n <= 0) return 0;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.p[i] = recv_ptrs[i];
  long long blocks = (n + 7) / 8;
  if (blocks > txh::sm_count() * 8) blocks = txh::sm_count() * 8;
  moe_dispatch_kernel<<<static_cast<int>(blocks), 256, 0, s>>>(static_cast<const __nv_bfloat16*>(src), ld, tok, k,
                                                               scale, dest_rank, dest_row, t, world, n, D, capacity,
                                                               status);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// out[t] = sum_j weights[t, j] * send_ptrs[dest_rank[t, j]][dest_row[t, j]] (weights null: plain sum), k <= 16.
// gathered (may be null) receives the k pulled rows of every token, [T * k, D].
extern "C" int tx_moe_combine_rows(void* const* send_ptrs, int world, const int* dest_rank, const int* dest_row,
                                   const float* weights, int k, void* out, long long ldo, void* gathered, long long T,
                                   int D, long long capacity, int* status, cudaStream_t s) {
  if (world < 1 || world > kMaxPeers || (D & 7) || (ldo & 7) || k < 1 || k > 16) return 1;
  if (T <= 0) return 0;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.p[i] = send_ptrs[i];
  const long long cap = static_cast<long long>(txh::sm_count()) * 16;
  const int grid = static_cast<int>(T < cap ? T : cap);
  auto* o = static_cast<__nv_bfloat16*>(out);
  auto* g = static_cast<__nv_bfloat16*>(gathered);
  if (k <= 2)
    moe_combine_kernel<2><<<grid, 128, 0, s>>>(t, world, dest_rank, dest_row, weights, k, o, ldo, g, T, D, capacity, status);
  else if (k <= 4)
    moe_combine_kernel<4><<<grid, 128, 0, s>>>(t, world, dest_rank, dest_row, weights, k, o, ldo, g, T, D, capacity, status);
  else if (k <= 8)
    moe_combine_kernel<8><<<grid, 128, 0, s>>>(t, world, dest_rank, dest_row, weights, k, o, ldo, g, T, D, capacity, status);
  else
    moe_combine_kernel<16><<<grid, 128, 0, s>>>(t, world, dest_rank, dest_row, weights, k, o, ldo, g, T, D, capacity, status);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}
