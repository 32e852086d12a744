// Collectives written as ordinary kernels over peer-mapped (NVLink / NVSwitch) memory.
//
// Every rank passes a table of device pointers - the same logical buffer on every rank of the
// group, each mapped into this process (CUDA IPC / symmetric memory). Kernels read or write the
// peers' buffers with plain 16-byte global loads and stores; NVSwitch gives every pair the full
// link bandwidth, so the access pattern simply rotates the peer order per rank to avoid all
// ranks hitting the same GPU at once.
//
//   tx_peer_barrier          : flag exchange in peer memory, bounded spin, error status on timeout
//   tx_reduce_scatter_sum_f32: out_shard[i] = sum_r grad_r[shard_off + i]   (+ sum of squares)
//   tx_adamw_allgather       : AdamW on this rank's fp32 master shard, then the refreshed bf16
//                              values are stored into every rank's parameter buffer
//   tx_peer_gather_copy      : pull a strided block from a peer (weight re-sharding)
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tx_host.h"

namespace {

constexpr int kMaxPeers = 16;

struct PeerTable {
  void* p[kMaxPeers];
};

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// flags.p[r] points at rank r's int32[kMaxPeers] flag row. Thread r of the single CTA tells peer r
// "rank `rank` reached epoch" and then waits until peer r has told us the same.
__global__ void peer_barrier_kernel(PeerTable flags, int rank, int world, int epoch, unsigned long long limit_ns,
                                    int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  st_release_sys(reinterpret_cast<int*>(flags.p[r]) + rank, epoch);
  const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + r;
  const uint64_t t0 = globaltimer_ns();
  while (ld_acquire_sys(mine) < epoch) {
    if (globaltimer_ns() - t0 > limit_ns) {
      atomicOr(status, 16);
      return;
    }
    __nanosleep(200);
  }
}

__global__ void __launch_bounds__(256)
reduce_scatter_sum_kernel(PeerTable grads, float* __restrict__ out, long long shard_off, long long n, int world,
                          int rank, float* __restrict__ sumsq_partials) {
  const long long n4 = n / 4;
  float ss = 0.f;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int k = 0; k < world; ++k) {
      int r = rank + k;
      if (r >= world) r -= world;
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + shard_off)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    reinterpret_cast<float4*>(out)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  if (sumsq_partials) {
    __shared__ float sh[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (blockDim.x >> 5); ++w) t += sh[w];
      sumsq_partials[blockIdx.x] = t;
    }
  }
}

// The same sum for use BESIDE compute kernels: few, long-lived CTAs (so they take a slot on a handful of SMs once
// and stay there instead of queueing wave after wave behind a persistent GEMM) with eight independent 16-byte
// loads per peer in flight per thread to keep the links busy from so few threads.
__global__ void __launch_bounds__(512)
reduce_scatter_sum_bg_kernel(PeerTable grads, float* __restrict__ out, long long shard_off, long long n, int world,
                             int rank) {
  constexpr int U = 8;
  const long long n4 = n / 4;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long base = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; base < n4; base += stride * U) {
    float4 acc[U];
#pragma unroll
    for (int u = 0; u < U; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < world; ++k) {
      int r = rank + k;
      if (r >= world) r -= world;
      const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + shard_off);
      float4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long i = base + u * stride;
        v[u] = i < n4 ? src[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) { acc[u].x += v[u].x; acc[u].y += v[u].y; acc[u].z += v[u].z; acc[u].w += v[u].w; }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long long i = base + u * stride;
      if (i < n4) reinterpret_cast<float4*>(out)[i] = acc[u];
    }
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;
};

// 8 elements per thread-iteration so the bf16 result is one 16-byte store per peer.
__global__ void __launch_bounds__(256)
adamw_allgather_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                       const float* __restrict__ grad, PeerTable params, long long shard_off, long long n,
                       AdamArgs a, const float* __restrict__ grad_scale, int world, int rank) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long long n8 = n / 8;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float p[8], mm[8], vv[8], g[8];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float4 p4 = reinterpret_cast<const float4*>(master)[2 * i + h];
      const float4 m4 = reinterpret_cast<const float4*>(m)[2 * i + h];
      const float4 v4 = reinterpret_cast<const float4*>(v)[2 * i + h];
      const float4 g4 = reinterpret_cast<const float4*>(grad)[2 * i + h];
      p[4 * h] = p4.x; p[4 * h + 1] = p4.y; p[4 * h + 2] = p4.z; p[4 * h + 3] = p4.w;
      mm[4 * h] = m4.x; mm[4 * h + 1] = m4.y; mm[4 * h + 2] = m4.z; mm[4 * h + 3] = m4.w;
      vv[4 * h] = v4.x; vv[4 * h + 1] = v4.y; vv[4 * h + 2] = v4.z; vv[4 * h + 3] = v4.w;
      g[4 * h] = g4.x; g[4 * h + 1] = g4.y; g[4 * h + 2] = g4.z; g[4 * h + 3] = g4.w;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float ge = g[e] * gs;
      mm[e] = a.beta1 * mm[e] + (1.f - a.beta1) * ge;
      vv[e] = a.beta2 * vv[e] + (1.f - a.beta2) * ge * ge;
      p[e] = p[e] - a.lr * ((mm[e] / a.bc1) / (sqrtf(vv[e] / a.bc2) + a.eps) + a.weight_decay * p[e]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      reinterpret_cast<float4*>(master)[2 * i + h] = make_float4(p[4 * h], p[4 * h + 1], p[4 * h + 2], p[4 * h + 3]);
      reinterpret_cast<float4*>(m)[2 * i + h] = make_float4(mm[4 * h], mm[4 * h + 1], mm[4 * h + 2], mm[4 * h + 3]);
      reinterpret_cast<float4*>(v)[2 * i + h] = make_float4(vv[4 * h], vv[4 * h + 1], vv[4 * h + 2], vv[4 * h + 3]);
    }
    uint4 packed;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(p[2 * e], p[2 * e + 1]);
    for (int k = 0; k < world; ++k) {
      int r = rank + k;
      if (r >= world) r -= world;
      reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[r]) + shard_off)[i] = packed;
    }
  }
}

// dst[row, 0:cols] = src_peer[row * src_ld + src_off ...]: 16-byte chunks, both sides bf16/any 2-byte type.
__global__ void __launch_bounds__(256)
peer_copy_2d_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long rows, long long cols16,
                    long long src_ld16, long long dst_ld16) {
  const long long total = rows * cols16;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / cols16, c = i - r * cols16;
    dst[r * dst_ld16 + c] = src[r * src_ld16 + c];
  }
}

// One 2-D block of a re-sharding plan: dst[r, 0:cols] = src[r, 0:cols] for r < rows, 2-byte elements.
// `src` / `dst` are absolute device addresses (either may be a peer mapping); leading dimensions in elements.
// `first_chunk` is the running count of 16-byte chunks (or of elements, for unaligned segments) before this one.
struct ReshardSeg {
  unsigned long long src, dst;
  long long rows, cols, src_ld, dst_ld;
  long long first_unit;      // prefix sum of work units
  int vec;                   // 1: every row start and `cols` are multiples of 8 elements -> 16-byte moves
  int pad;
};

// Walks a whole plan in one launch: work unit u belongs to the segment found by binary search in the
// prefix sums; a unit is a 16-byte chunk of a row (vec) or a single element.
__global__ void __launch_bounds__(256)
reshard_copy_kernel(const ReshardSeg* __restrict__ segs, int n_segs, long long total_units) {
  for (long long u = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; u < total_units;
       u += static_cast<long long>(gridDim.x) * blockDim.x) {
    int lo = 0, hi = n_segs - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (segs[mid].first_unit <= u) lo = mid; else hi = mid - 1;
    }
    const ReshardSeg sg = segs[lo];
    const long long k = u - sg.first_unit;
    if (sg.vec) {
      const long long per_row = sg.cols >> 3;
      const long long r = k / per_row, c = k - r * per_row;
      const uint4* s = reinterpret_cast<const uint4*>(sg.src) + ((r * sg.src_ld) >> 3) + c;
      uint4* d = reinterpret_cast<uint4*>(sg.dst) + ((r * sg.dst_ld) >> 3) + c;
      *d = *s;
    } else {
      const long long r = k / sg.cols, c = k - r * sg.cols;
      reinterpret_cast<unsigned short*>(sg.dst)[r * sg.dst_ld + c] =
          reinterpret_cast<const unsigned short*>(sg.src)[r * sg.src_ld + c];
    }
  }
}

// Publishes a finished copy: version word = value, after everything the stream did before.
__global__ void publish_version_kernel(int* version, int value) {
  __threadfence_system();
  *reinterpret_cast<volatile int*>(version) = value;
}

inline int grid_for(long long items, int threads, int cap_per_sm) {
  long long b = (items + threads - 1) / threads;
  const long long cap = static_cast<long long>(txh::sm_count()) * cap_per_sm;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace

extern "C" int tx_peer_barrier(void* const* flag_rows, int rank, int world, int epoch, long long limit_ms,
                               int* status, cudaStream_t s) {
  if (world > kMaxPeers) return 1;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.p[i] = flag_rows[i];
  peer_barrier_kernel<<<1, 32, 0, s>>>(t, rank, world, epoch, static_cast<unsigned long long>(limit_ms) * 1000000ull,
                                       status);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// Number of CTAs (and of floats in `sumsq_partials`) the reduce-scatter kernel uses.
extern "C" int tx_reduce_scatter_grid() { return txh::sm_count() * 4; }

extern "C" int tx_reduce_scatter_sum_f32(void* const* grad_ptrs, float* out_shard, long long shard_off, long long n,
                                         int world, int rank, float* sumsq_partials, cudaStream_t s) {
  if (world > kMaxPeers || (n & 3) || (shard_off & 3)) return 1;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.p[i] = grad_ptrs[i];
  reduce_scatter_sum_kernel<<<tx_reduce_scatter_grid(), 256, 0, s>>>(t, out_shard, shard_off, n, world, rank,
                                                                     sumsq_partials);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// Background variant (no sum of squares): `ctas` CTAs of 512 threads, meant for a side stream next to compute.
extern "C" int tx_reduce_scatter_sum_f32_bg(void* const* grad_ptrs, float* out_shard, long long shard_off, long long n,
                                            int world, int rank, int ctas, cudaStream_t s) {
  if (world > kMaxPeers || (n & 3) || (shard_off & 3) || ctas <= 0) return 1;
  if (n == 0) return 0;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.p[i] = grad_ptrs[i];
  reduce_scatter_sum_bg_kernel<<<ctas, 512, 0, s>>>(t, out_shard, shard_off, n, world, rank);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

extern "C" int tx_adamw_allgather(float* master, float* m, float* v, const float* grad, void* const* param_ptrs,
                                  long long shard_off, long long n, float lr, float beta1, float beta2, float eps,
                                  float weight_decay, float bc1, float bc2, const float* grad_scale, int world,
                                  int rank, cudaStream_t s) {
  if (world > kMaxPeers || (n & 7) || (shard_off & 7)) return 1;
  PeerTable t;
  for (int i = 0; i < world; ++i) t.p[i] = param_ptrs[i];
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bc1, bc2};
  adamw_allgather_kernel<<<grid_for(n / 8, 256, 8), 256, 0, s>>>(master, m, v, grad, t, shard_off, n, a, grad_scale,
                                                                world, rank);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// Copies a [rows, cols] block of 2-byte elements; pointers and leading dimensions (in elements) must be
// multiples of 8 elements (16 bytes). Either pointer may be peer memory.
extern "C" int tx_peer_copy_2d(const void* src, void* dst, long long rows, long long cols, long long src_ld,
                               long long dst_ld, cudaStream_t s) {
  if ((cols & 7) || (src_ld & 7) || (dst_ld & 7)) return 1;
  if (rows <= 0 || cols <= 0) return 0;
  peer_copy_2d_kernel<<<grid_for(rows * (cols / 8), 256, 8), 256, 0, s>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), rows, cols / 8, src_ld / 8, dst_ld / 8);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// Executes a re-sharding plan (`n_segs` ReshardSeg records in device memory, `total_units` = the last prefix sum +
// the last segment's units) in one launch, then - when `version` is given - stores `version_value` there, ordered
// after the copies, so a reader that polls the word knows the whole replica is in place. Sources may be peer
// mappings (trainer rank -> rollout rank over NVLink); plain loads and stores only.
extern "C" int tx_reshard_copy(const void* segs, int n_segs, long long total_units, int* version, int version_value,
                               cudaStream_t s) {
  if (n_segs < 0 || total_units < 0) return 1;
  if (n_segs > 0 && total_units > 0) {
    reshard_copy_kernel<<<grid_for(total_units, 256, 8), 256, 0, s>>>(static_cast<const ReshardSeg*>(segs), n_segs,
                                                                     total_units);
    if (cudaGetLastError() != cudaSuccess) return 400;
  }
  if (version) publish_version_kernel<<<1, 1, 0, s>>>(version, version_value);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

extern "C" int tx_reshard_seg_bytes() { return static_cast<int>(sizeof(ReshardSeg)); }
