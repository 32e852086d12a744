// Selective log-softmax over a block of logits: per row the log-probability of one target
// id, the log-sum-exp and (optionally) the entropy, in fp32; and the matching backward that
// overwrites the logits block with d(loss)/d(logits) in bf16, ready to feed the two
// lm-head gradient GEMMs. The same kernels serve the trainer, the reference policy and the
// rollout sampler, so their per-token log-probabilities share one reduction order.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

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

// One CTA per row. logits: [T, ld] (V valid columns). z = logit * inv_temp (soft-capped first
// when softcap > 0: cap * tanh(logit / cap)).
template <typename LT>
__global__ void __launch_bounds__(kThreads)
logprob_fwd_kernel(const LT* __restrict__ logits, long long ldl, const int* __restrict__ targets,
                   float* __restrict__ logp, float* __restrict__ lse_out, float* __restrict__ entropy, int T,
                   int V, float inv_temp, float softcap) {
  __shared__ Acc sh[kThreads / 32];
  const int row = blockIdx.x;
  if (row >= T) return;
  const LT* lr = logits + static_cast<long long>(row) * ldl;
  Acc a{-INFINITY, 0.f, 0.f};
  for (int j = threadIdx.x; j < V; j += kThreads) {
    float z = ld<LT>(lr + j);
    if (softcap > 0.f) z = softcap * tanhf(z / softcap);
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
    float zt = 0.f;
    if (tgt >= 0 && tgt < V) {
      zt = ld<LT>(lr + tgt);
      if (softcap > 0.f) zt = softcap * tanhf(zt / softcap);
      zt *= inv_temp;
    }
    logp[row] = (tgt >= 0 && tgt < V) ? zt - lse : 0.f;
    if (lse_out) lse_out[row] = lse;
    if (entropy) entropy[row] = lse - r.sz / r.s;
  }
}

// dlogits[j] = inv_temp * dcap_j * ( g_logp * (1[j==tgt] - p_j) - g_ent * p_j * (z_j - lse + H) )
// written as bf16 into dl (row stride ldd). p_j = exp(z_j - lse).
template <typename LT>
__global__ void __launch_bounds__(kThreads)
logprob_bwd_kernel(const LT* __restrict__ logits, long long ldl, const int* __restrict__ targets,
                   const float* __restrict__ lse_in, const float* __restrict__ entropy_in,
                   const float* __restrict__ g_logp, const float* __restrict__ g_ent,
                   __nv_bfloat16* __restrict__ dl, long long ldd, int T, int V, int V_pad, float inv_temp,
                   float softcap) {
  const int row = blockIdx.x;
  if (row >= T) return;
  const LT* lr = logits + static_cast<long long>(row) * ldl;
  __nv_bfloat16* dr = dl + static_cast<long long>(row) * ldd;
  const float lse = lse_in[row];
  const float gl = g_logp ? g_logp[row] : 0.f;
  const float ge = g_ent ? g_ent[row] : 0.f;
  const float H = (g_ent && entropy_in) ? entropy_in[row] : 0.f;
  const int tgt = targets[row];
  for (int j = threadIdx.x; j < V_pad; j += kThreads) {
    float d = 0.f;
    if (j < V) {
      const float raw = ld<LT>(lr + j);
      float z = raw, dcap = 1.f;
      if (softcap > 0.f) {
        const float th = tanhf(raw / softcap);
        z = softcap * th;
        dcap = 1.f - th * th;
      }
      z *= inv_temp;
      const float p = __expf(z - lse);
      d = gl * ((j == tgt ? 1.f : 0.f) - p);
      if (ge != 0.f) d -= ge * p * (z - lse + H);
      d *= inv_temp * dcap;
    }
    dr[j] = __float2bfloat16_rn(d);
  }
}

}  // namespace

// logits_fp32 != 0: logits are float32, else bf16. ldl is the row stride in elements.
extern "C" int tx_logprob_fwd(const void* logits, int logits_fp32, long long ldl, const int* targets, float* logp,
                              float* lse, float* entropy, int T, int V, float inv_temp, float softcap,
                              cudaStream_t s) {
  if (T <= 0) return 0;
  if (logits_fp32)
    logprob_fwd_kernel<float><<<T, kThreads, 0, s>>>((const float*)logits, ldl, targets, logp, lse, entropy, T, V,
                                                     inv_temp, softcap);
  else
    logprob_fwd_kernel<__nv_bfloat16><<<T, kThreads, 0, s>>>((const __nv_bfloat16*)logits, ldl, targets, logp,
                                                             lse, entropy, T, V, inv_temp, softcap);
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
  if (logits_fp32)
    logprob_bwd_kernel<float><<<T, kThreads, 0, s>>>((const float*)logits, ldl, targets, lse, entropy, g_logp,
                                                     g_ent, (__nv_bfloat16*)dl, ldd, T, V, V_pad, inv_temp, softcap);
  else
    logprob_bwd_kernel<__nv_bfloat16><<<T, kThreads, 0, s>>>((const __nv_bfloat16*)logits, ldl, targets, lse,
                                                             entropy, g_logp, g_ent, (__nv_bfloat16*)dl, ldd, T, V,
                                                             V_pad, inv_temp, softcap);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}
