// Bandwidth-bound kernels: gated activations (SwiGLU / GeGLU), embedding gather and its
// scatter-add backward, the flat AdamW update with fp32 master weights, fp32 gradient norm
// with clipping, and a few cast / scale helpers. 16-byte vector accesses throughout.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tx_debug.cuh"
#include "tx_host.h"

TX_DEBUG_UNIT(elementwise)

namespace {

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&f)[8]) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float dsilu_f(float x) {
  const float s = 1.f / (1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}
// tanh-approximated GELU, the form the Gemma family uses.
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float dgelu_tanh_f(float x) {
  const float k = 0.7978845608028654f;
  const float u = k * (x + 0.044715f * x * x * x);
  const float t = tanhf(u);
  return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * k * (1.f + 3.f * 0.044715f * x * x);
}

// gu is [T, 2F] = [gate | up]; out[T, F] = act(gate) * up.
template <bool GELU>
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                               long long T, int F) {
  const int fv = F / 8;
  const long long total = T * fv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / fv;
    const int c = static_cast<int>(i - t * fv) * 8;
    float g[8], u[8], o[8];
    load8(gu + t * 2 * F + c, g);
    load8(gu + t * 2 * F + F + c, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = (GELU ? gelu_tanh_f(g[e]) : silu_f(g[e])) * u[e];
    store8(out + t * F + c, o);
  }
}

template <bool GELU>
__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dout,
                               __nv_bfloat16* __restrict__ dgu, long long T, int F) {
  const int fv = F / 8;
  const long long total = T * fv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / fv;
    const int c = static_cast<int>(i - t * fv) * 8;
    float g[8], u[8], d[8], dg[8], du[8];
    load8(gu + t * 2 * F + c, g);
    load8(gu + t * 2 * F + F + c, u);
    load8(dout + t * F + c, d);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float a = GELU ? gelu_tanh_f(g[e]) : silu_f(g[e]);
      const float da = GELU ? dgelu_tanh_f(g[e]) : dsilu_f(g[e]);
      dg[e] = d[e] * u[e] * da;
      du[e] = d[e] * a;
    }
    store8(dgu + t * 2 * F + c, dg);
    store8(dgu + t * 2 * F + F + c, du);
  }
}

// out[t, :] = table[ids[t], :] * scale
__global__ void embedding_fwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                     __nv_bfloat16* __restrict__ out, long long T, int D, int V, float scale) {
  const int dv = D / 8;
  const long long total = T * dv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / dv;
    const int c = static_cast<int>(i - t * dv) * 8;
    int id = ids[t];
    TX_DEBUG_CHECK(id >= 0 && id < V, TX_DBG_TOKEN_ID, id, V);
    id = id < 0 ? 0 : (id >= V ? V - 1 : id);
    float v[8];
    load8(table + static_cast<long long>(id) * D + c, v);
    if (scale != 1.f) {
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] *= scale;
    }
    store8(out + t * D + c, v);
  }
}

// grad_table[ids[t], :] += dout[t, :] * scale   (fp32 accumulation with atomics)
__global__ void embedding_bwd_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ dout,
                                     float* __restrict__ grad_table, long long T, int D, int V, float scale) {
  const int dv = D / 8;
  const long long total = T * dv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long t = i / dv;
    const int c = static_cast<int>(i - t * dv) * 8;
    const int id = ids[t];
    if (id < 0 || id >= V) continue;
    float v[8];
    load8(dout + t * D + c, v);
    float* dst = grad_table + static_cast<long long>(id) * D + c;
#pragma unroll
    for (int e = 0; e < 8; ++e) atomicAdd(dst + e, v[e] * scale);
  }
}

// ---- optimizer -----------------------------------------------------------------------
struct AdamArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;  // bc = 1 - beta^t
};

// One fused pass: g = grad * (*grad_scale); AdamW on the fp32 master copy; refresh the bf16
// compute copy; optionally zero the gradient for the next accumulation window.
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             float* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, long long n,
                             AdamArgs a, const float* __restrict__ grad_scale, int zero_grad) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float4 g4 = reinterpret_cast<float4*>(grad)[i];
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float* g = reinterpret_cast<float*>(&g4);
    float* p = reinterpret_cast<float*>(&p4);
    float* mm = reinterpret_cast<float*>(&m4);
    float* vv = reinterpret_cast<float*>(&v4);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float ge = g[e] * gs;
      mm[e] = a.beta1 * mm[e] + (1.f - a.beta1) * ge;
      vv[e] = a.beta2 * vv[e] + (1.f - a.beta2) * ge * ge;
      const float mhat = mm[e] / a.bc1;
      const float vhat = vv[e] / a.bc2;
      p[e] = p[e] - a.lr * (mhat / (sqrtf(vhat) + a.eps) + a.weight_decay * p[e]);
    }
    reinterpret_cast<float4*>(master)[i] = p4;
    reinterpret_cast<float4*>(m)[i] = m4;
    reinterpret_cast<float4*>(v)[i] = v4;
    if (zero_grad) reinterpret_cast<float4*>(grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (param_bf16) {
      __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(param_bf16) + 2 * i;
      o[0] = __floats2bfloat162_rn(p[0], p[1]);
      o[1] = __floats2bfloat162_rn(p[2], p[3]);
    }
  }
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const long long i = n4 * 4 + threadIdx.x;
    const float ge = grad[i] * gs;
    const float m1 = a.beta1 * m[i] + (1.f - a.beta1) * ge;
    const float v1 = a.beta2 * v[i] + (1.f - a.beta2) * ge * ge;
    const float pn = master[i] - a.lr * ((m1 / a.bc1) / (sqrtf(v1 / a.bc2) + a.eps) + a.weight_decay * master[i]);
    m[i] = m1; v[i] = v1; master[i] = pn;
    if (zero_grad) grad[i] = 0.f;
    if (param_bf16) param_bf16[i] = __float2bfloat16_rn(pn);
  }
}

__global__ void sumsq_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partials) {
  __shared__ float sh[32];
  float s = 0.f;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < (n & 3)) {
    const float t = x[n4 * 4 + threadIdx.x];
    s += t * t;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (threadIdx.x == 0) partials[blockIdx.x] = s;
  }
}

// out[0] += sum(partials) (in a fixed order). Launched with one block of 256 threads.
__global__ void fold_partials_kernel(const float* __restrict__ partials, int P, float* __restrict__ out,
                                     int accumulate) {
  __shared__ double sh[256];
  double s = 0.0;
  for (int i = threadIdx.x; i < P; i += 256) s += partials[i];
  sh[threadIdx.x] = s;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) sh[threadIdx.x] += sh[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = (accumulate ? out[0] : 0.f) + static_cast<float>(sh[0]);
}

// Given sumsq (of the *unscaled* accumulated gradient) and inv_denom (device scalars), writes
//   norm_out  = sqrt(sumsq) * inv_denom                     (the fp32 global gradient norm)
//   scale_out = inv_denom * min(1, max_norm / (norm + 1e-6)) (what AdamW multiplies grads by)
__global__ void clip_scale_kernel(const float* __restrict__ sumsq, const float* __restrict__ inv_denom,
                                  float max_norm, float* __restrict__ norm_out, float* __restrict__ scale_out) {
  const float inv = inv_denom ? *inv_denom : 1.f;
  const float norm = sqrtf(*sumsq) * inv;
  float clip = 1.f;
  if (max_norm > 0.f && norm > max_norm) clip = max_norm / (norm + 1e-6f);
  *norm_out = norm;
  *scale_out = inv * clip;
}

__global__ void cast_f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                        long long n) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16_rn(in[i]);
}

// acc[i] += x[i] (bf16 -> fp32 accumulate), used when a bf16 gradient is folded into the fp32 buffer.
__global__ void accum_bf16_into_f32_kernel(const __nv_bfloat16* __restrict__ x, float* __restrict__ acc,
                                           long long n, float scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    acc[i] += __bfloat162float(x[i]) * scale;
}

inline int grid_for(long long work_items, int threads) {
  long long b = (work_items + threads - 1) / threads;
  const long long cap = static_cast<long long>(txh::sm_count()) * 16;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace

#define TX_OK() (cudaGetLastError() == cudaSuccess ? 0 : 400)

extern "C" int tx_glu_fwd(const void* gu, void* out, long long T, int F, int gelu, cudaStream_t s) {
  if (F % 8) return 1;
  if (T <= 0) return 0;
  const int g = grid_for(T * (F / 8), 256);
  if (gelu) glu_fwd_kernel<true><<<g, 256, 0, s>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, F);
  else      glu_fwd_kernel<false><<<g, 256, 0, s>>>((const __nv_bfloat16*)gu, (__nv_bfloat16*)out, T, F);
  return TX_OK();
}

extern "C" int tx_glu_bwd(const void* gu, const void* dout, void* dgu, long long T, int F, int gelu,
                          cudaStream_t s) {
  if (F % 8) return 1;
  if (T <= 0) return 0;
  const int g = grid_for(T * (F / 8), 256);
  if (gelu) glu_bwd_kernel<true><<<g, 256, 0, s>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, T, F);
  else      glu_bwd_kernel<false><<<g, 256, 0, s>>>((const __nv_bfloat16*)gu, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dgu, T, F);
  return TX_OK();
}

extern "C" int tx_embedding_fwd(const int* ids, const void* table, void* out, long long T, int D, int V,
                                float scale, cudaStream_t s) {
  if (D % 8) return 1;
  if (T <= 0) return 0;
  embedding_fwd_kernel<<<grid_for(T * (D / 8), 256), 256, 0, s>>>(ids, (const __nv_bfloat16*)table,
                                                                  (__nv_bfloat16*)out, T, D, V, scale);
  return TX_OK();
}

extern "C" int tx_embedding_bwd(const int* ids, const void* dout, float* grad_table, long long T, int D, int V,
                                float scale, cudaStream_t s) {
  if (D % 8) return 1;
  if (T <= 0) return 0;
  embedding_bwd_kernel<<<grid_for(T * (D / 8), 256), 256, 0, s>>>(ids, (const __nv_bfloat16*)dout, grad_table,
                                                                  T, D, V, scale);
  return TX_OK();
}

extern "C" int tx_adamw(float* master, float* m, float* v, float* grad, void* param_bf16, long long n, float lr,
                        float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2,
                        const float* grad_scale, int zero_grad, cudaStream_t s) {
  if (n <= 0) return 0;
  AdamArgs a{lr, beta1, beta2, eps, weight_decay, bc1, bc2};
  adamw_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, s>>>(master, m, v, grad, (__nv_bfloat16*)param_bf16, n, a,
                                                         grad_scale, zero_grad);
  return TX_OK();
}

// Scratch: `partials` must hold tx_sumsq_partials() floats.
extern "C" int tx_sumsq_partials() { return txh::sm_count() * 8; }

extern "C" int tx_sumsq(const float* x, long long n, float* partials, float* out, int accumulate,
                        cudaStream_t s) {
  int g = grid_for(n / 4 + 1, 256);
  if (g > tx_sumsq_partials()) g = tx_sumsq_partials();
  sumsq_partial_kernel<<<g, 256, 0, s>>>(x, n, partials);
  fold_partials_kernel<<<1, 256, 0, s>>>(partials, g, out, accumulate);
  return TX_OK();
}

extern "C" int tx_clip_scale(const float* sumsq, const float* inv_denom, float max_norm, float* norm_out,
                             float* scale_out, cudaStream_t s) {
  clip_scale_kernel<<<1, 1, 0, s>>>(sumsq, inv_denom, max_norm, norm_out, scale_out);
  return TX_OK();
}

extern "C" int tx_cast_f32_bf16(const float* in, void* out, long long n, cudaStream_t s) {
  if (n <= 0) return 0;
  cast_f32_to_bf16_kernel<<<grid_for(n, 256), 256, 0, s>>>(in, (__nv_bfloat16*)out, n);
  return TX_OK();
}

extern "C" int tx_accum_bf16_f32(const void* x, float* acc, long long n, float scale, cudaStream_t s) {
  if (n <= 0) return 0;
  accum_bf16_into_f32_kernel<<<grid_for(n, 256), 256, 0, s>>>((const __nv_bfloat16*)x, acc, n, scale);
  return TX_OK();
}
