// Selective log-softmax over a block of logits: per row the log-probability of one target
// id, the log-sum-exp and (optionally) the entropy, in fp32; and the matching backward that
// overwrites the logits block with d(loss)/d(logits) in bf16, ready to feed the two
// lm-head gradient GEMMs. The same kernels serve the trainer, the reference policy and the
// rollout sampler, so their per-token log-probabilities share one reduction order.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "tx_debug.cuh"

TX_DEBUG_UNIT(logprob)

namespace {

constexpr int kThreads = 512;

struct Acc {
  float m;   // running max
  float s;   // sum exp(z - m)
  float sz;  // sum exp(z - m) * z   (for the entropy)
};

__device__ __forceinline__ Acc acc_merge(const Acc& a, const Acc& b) {
  Acc r;
  r.m = fmaxf(a.m, b.m);
  const float ea = (a.m == -INFINITY) ? 0.f : __expf(a.m - r.m);
  const float eb = (b.m == -INFINITY) ? 0.f : __expf(b.m - r.m);
  r.s = a.s * ea + b.s * eb;
  r.sz = a.sz * ea + b.sz * eb;
  return r;
}

__device__ __forceinline__ void acc_push(Acc& a, float z) {
  if (z > a.m) {
    const float e = (a.m == -INFINITY) ? 0.f : __expf(a.m - z);
    a.s = a.s * e + 1.f;
    a.sz = a.sz * e + z;
    a.m = z;
  } else {
    const float e = __expf(z - a.m);
    a.s += e;
    a.sz += e * z;
  }
}

template <typename T>
__device__ __forceinline__ float ld(const T* p);
template <>
__device__ __forceinline__ float ld<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

// Eight consecutive logits starting at an element offset that is a multiple of 8 from a
// 16-byte aligned row base.
__device__ __forceinline__ void ld8(const float* p, float (&z)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  z[0] = a.x; z[1] = a.y; z[2] = a.z; z[3] = a.w; z[4] = b.x; z[5] = b.y; z[6] = b.z; z[7] = b.w;
}
__device__ __forceinline__ void ld8(const __nv_bfloat16* p, float (&z)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    z[2 * i] = f.x;
    z[2 * i + 1] = f.y;
  }
}

// Folds eight values into the running (max, sum, sum*z) with one rescale.
__device__ __forceinline__ void acc_push8(Acc& a, const float (&z)[8]) {
  float vm = z[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) vm = fmaxf(vm, z[i]);
  const float mn = fmaxf(a.m, vm);
  const float e = (a.m == -INFINITY) ? 0.f : __expf(a.m - mn);
  float s = 0.f, sz = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float w = __expf(z[i] - mn);
    s += w;
    sz += w * z[i];
  }
  a.s = a.s * e + s;
  a.sz = a.sz * e + sz;
  a.m = mn;
}

// One CTA per row. logits: [T, ld] (V valid columns). z = logit * inv_temp (soft-capped first
// when softcap > 0: cap * tanh(logit / cap)). `vec` says rows are 16-byte aligned, so the body
// runs on 8-element vectors, two in flight per thread; the ragged tail is scalar.
template <typename LT>
__global__ void __launch_bounds__(kThreads)
logprob_fwd_kernel(const LT* __restrict__ logits, long long ldl, const int* __restrict__ targets,
                   float* __restrict__ logp, float* __restrict__ lse_out, float* __restrict__ entropy, int T,
                   int V, float inv_temp, float softcap, int vec) {
  __shared__ Acc sh[kThreads / 32];
  const int row = blockIdx.x;
  if (row >= T) return;
  const LT* lr = logits + static_cast<long long>(row) * ldl;
  Acc a{-INFINITY, 0.f, 0.f};
  const int V8 = vec ? (V & ~7) : 0;
  const bool cap = softcap > 0.f;
  const float inv_cap = cap ? 1.f / softcap : 0.f;
  int j = threadIdx.x * 8;
  for (; j + kThreads * 8 < V8; j += 2 * kThreads * 8) {
    float z0[8], z1[8];
    ld8(lr + j, z0);
    ld8(lr + j + kThreads * 8, z1);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (cap) { z0[i] = softcap * tanhf(z0[i] * inv_cap); z1[i] = softcap * tanhf(z1[i] * inv_cap); }
      z0[i] *= inv_temp;
      z1[i] *= inv_temp;
    }
    acc_push8(a, z0);
    acc_push8(a, z1);
  }
  if (j < V8) {
    float z0[8];
    ld8(lr + j, z0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (cap) z0[i] = softcap * tanhf(z0[i] * inv_cap);
      z0[i] *= inv_temp;
    }
    acc_push8(a, z0);
  }
  for (int t = V8 + threadIdx.x; t < V; t += kThreads) {
    float z = ld<LT>(lr + t);
    if (cap) z = softcap * tanhf(z * inv_cap);
    acc_push(a, z * inv_temp);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Acc b;
    b.m = __shfl_xor_sync(0xffffffffu, a.m, o);
    b.s = __shfl_xor_sync(0xffffffffu, a.s, o);
    b.sz = __shfl_xor_sync(0xffffffffu, a.sz, o);
    a = acc_merge(a, b);
  }
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = a;
  __syncthreads();
  if (threadIdx.x == 0) {
    Acc r = sh[0];
    for (int w = 1; w < kThreads / 32; ++w) r = acc_merge(r, sh[w]);
    const float lse = r.m + logf(r.s);
    const int tgt = targets[row];
    TX_DEBUG_CHECK(tgt >= 0 && tgt < V, TX_DBG_TARGET_ID, tgt, V);
    float zt = 0.f;
    if (tgt >= 0 && tgt < V) {
      zt = ld<LT>(lr + tgt);
      if (cap) zt = softcap * tanhf(zt * inv_cap);
      zt *= inv_temp;
    }
    logp[row] = (tgt >= 0 && tgt < V) ? zt - lse : 0.f;
    if (lse_out) lse_out[row] = lse;
    if (entropy) entropy[row] = lse - r.sz / r.s;
  }
}

__device__ __forceinline__ float dlogit(float raw, int j, int tgt, float lse, float gl, float ge, float H,
                                        float inv_temp, float softcap) {
  float z = raw, dcap = 1.f;
  if (softcap > 0.f) {
    const float th = tanhf(raw / softcap);
    z = softcap * th;
    dcap = 1.f - th * th;
  }
  z *= inv_temp;
  const float p = __expf(z - lse);
  float d = gl * ((j == tgt ? 1.f : 0.f) - p);
  if (ge != 0.f) d -= ge * p * (z - lse + H);
  return d * inv_temp * dcap;
}

// dlogits[j] = inv_temp * dcap_j * ( g_logp * (1[j==tgt] - p_j) - g_ent * p_j * (z_j - lse + H) )
// written as bf16 into dl (row stride ldd). p_j = exp(z_j - lse). With `vec` (rows of both
// buffers 16-byte aligned) eight elements are read and written per thread and iteration.
template <typename LT>
__global__ void __launch_bounds__(kThreads)
logprob_bwd_kernel(const LT* __restrict__ logits, long long ldl, const int* __restrict__ targets,
                   const float* __restrict__ lse_in, const float* __restrict__ entropy_in,
                   const float* __restrict__ g_logp, const float* __restrict__ g_ent,
                   __nv_bfloat16* __restrict__ dl, long long ldd, int T, int V, int V_pad, float inv_temp,
                   float softcap, int vec) {
  const int row = blockIdx.x;
  if (row >= T) return;
  const LT* lr = logits + static_cast<long long>(row) * ldl;
  __nv_bfloat16* dr = dl + static_cast<long long>(row) * ldd;
  const float lse = lse_in[row];
  const float gl = g_logp ? g_logp[row] : 0.f;
  const float ge = g_ent ? g_ent[row] : 0.f;
  const float H = (g_ent && entropy_in) ? entropy_in[row] : 0.f;
  const int tgt = targets[row];
  const int V8 = vec ? (V & ~7) : 0;
  for (int j = threadIdx.x * 8; j < V8; j += kThreads * 8) {
    float z[8];
    ld8(lr + j, z);
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
      const float d0 = dlogit(z[i], j + i, tgt, lse, gl, ge, H, inv_temp, softcap);
      const float d1 = dlogit(z[i + 1], j + i + 1, tgt, lse, gl, ge, H, inv_temp, softcap);
      __nv_bfloat162 h = __floats2bfloat162_rn(d0, d1);
      ow[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(dr + j) = o;
  }
  for (int j = V8 + threadIdx.x; j < V_pad; j += kThreads) {
    float d = 0.f;
    if (j < V) d = dlogit(ld<LT>(lr + j), j, tgt, lse, gl, ge, H, inv_temp, softcap);
    dr[j] = __float2bfloat16_rn(d);
  }
}

}  // namespace

// logits_fp32 != 0: logits are float32, else bf16. ldl is the row stride in elements.
extern "C" int tx_logprob_fwd(const void* logits, int logits_fp32, long long ldl, const int* targets, float* logp,
                              float* lse, float* entropy, int T, int V, float inv_temp, float softcap,
                              cudaStream_t s) {
  if (T <= 0) return 0;
  const long long esz = logits_fp32 ? 4 : 2;
  const int vec = (reinterpret_cast<uintptr_t>(logits) % 16 == 0) && ((ldl * esz) % 16 == 0);
  if (logits_fp32)
    logprob_fwd_kernel<float><<<T, kThreads, 0, s>>>((const float*)logits, ldl, targets, logp, lse, entropy, T, V,
                                                     inv_temp, softcap, vec);
  else
    logprob_fwd_kernel<__nv_bfloat16><<<T, kThreads, 0, s>>>((const __nv_bfloat16*)logits, ldl, targets, logp,
                                                             lse, entropy, T, V, inv_temp, softcap, vec);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// Writes bf16 dlogits [T, V_pad] (columns V..V_pad-1 zero). dl may alias `logits` only when
// the logits are bf16 with the same stride (each element is read before it is overwritten by
// the same thread).
extern "C" int tx_logprob_bwd(const void* logits, int logits_fp32, long long ldl, const int* targets,
                              const float* lse, const float* entropy, const float* g_logp, const float* g_ent,
                              void* dl, long long ldd, int T, int V, int V_pad, float inv_temp, float softcap,
                              cudaStream_t s) {
  if (T <= 0) return 0;
  const long long esz = logits_fp32 ? 4 : 2;
  const int vec = (reinterpret_cast<uintptr_t>(logits) % 16 == 0) && ((ldl * esz) % 16 == 0) &&
                  (reinterpret_cast<uintptr_t>(dl) % 16 == 0) && (ldd % 8 == 0);
  if (logits_fp32)
    logprob_bwd_kernel<float><<<T, kThreads, 0, s>>>((const float*)logits, ldl, targets, lse, entropy, g_logp,
                                                     g_ent, (__nv_bfloat16*)dl, ldd, T, V, V_pad, inv_temp, softcap,
                                                     vec);
  else
    logprob_bwd_kernel<__nv_bfloat16><<<T, kThreads, 0, s>>>((const __nv_bfloat16*)logits, ldl, targets, lse,
                                                             entropy, g_logp, g_ent, (__nv_bfloat16*)dl, ldd, T, V,
                                                             V_pad, inv_temp, softcap, vec);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}
