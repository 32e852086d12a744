// RMSNorm (forward / backward, optional fused residual add), per-head q/k RMSNorm fused
// with rotary embedding, and plain rotary embedding. All bandwidth-bound: 16-byte vector
// accesses, fp32 math, one pass over HBM per tensor.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tx_host.h"

namespace {

constexpr int kNormThreads = 256;
constexpr int kMaxVec = 4;  // per-thread vectors of 8 bf16: D <= 256 * 8 * 4 = 8192

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? sh[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) sh[0] = t;
  }
  __syncthreads();
  return sh[0];
}

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

// y = x_sum * rsqrt(mean(x_sum^2) + eps) * (w + w_offset), x_sum = x (+ res).
// When res != nullptr the sum is also written to sum_out (the new residual stream).
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd_out, int T, int D, float eps,
                   float w_offset) {
  __shared__ float sh[32];
  // A successor launched with programmatic stream serialization (the decode GEMM) may start its set-up and weight
  // prefetch now; it still waits for this grid to finish before it reads y. No effect on ordinary successors.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int nvec = D / 8;
  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const __nv_bfloat16* xr = x + static_cast<size_t>(row) * D;
    float v[kMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      if (c < nvec) {
        load8(xr + c * 8, v[i]);
        if (res) {
          float r[8];
          load8(res + static_cast<size_t>(row) * D + c * 8, r);
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] += r[e];
          // round to the stored precision so forward and recompute see the same stream
#pragma unroll
          for (int e = 0; e < 8; ++e) v[i][e] = __bfloat162float(__float2bfloat16_rn(v[i][e]));
          store8(sum_out + static_cast<size_t>(row) * D + c * 8, v[i]);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += v[i][e] * v[i][e];
      }
    }
    ss = block_sum(ss, sh);
    const float rstd = rsqrtf(ss / D + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      if (c < nvec) {
        float wv[8], o[8];
        load8(w + c * 8, wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = v[i][e] * rstd * (wv[e] + w_offset);
        store8(y + static_cast<size_t>(row) * D + c * 8, o);
      }
    }
  }
}

// dx = rstd * (g - xhat * mean(g * xhat)) (+ dres), g = dy * (w + w_offset), xhat = x * rstd.
// Per-CTA partial dw sums go to dw_partial[gridDim.x, D]; a second kernel folds them.
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int T, int D, float eps, float w_offset) {
  __shared__ float sh[32];
  const int nvec = D / 8;
  float dw_acc[kMaxVec][8];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i)
#pragma unroll
    for (int e = 0; e < 8; ++e) dw_acc[i][e] = 0.f;

  for (int row = blockIdx.x; row < T; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * D;
    float xv[kMaxVec][8], gv[kMaxVec][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      if (c < nvec) {
        load8(x + off + c * 8, xv[i]);
        load8(dy + off + c * 8, gv[i]);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += xv[i][e] * xv[i][e];
      }
    }
    float rstd;
    if (rstd_in) {
      rstd = rstd_in[row];
    } else {
      ss = block_sum(ss, sh);
      rstd = rsqrtf(ss / D + eps);
    }
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      if (c < nvec) {
        float wv[8];
        load8(w + c * 8, wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float xh = xv[i][e] * rstd;
          dw_acc[i][e] += gv[i][e] * xh;
          gv[i][e] *= (wv[e] + w_offset);
          dot += gv[i][e] * xh;
          xv[i][e] = xh;
        }
      }
    }
    dot = block_sum(dot, sh) / D;
#pragma unroll
    for (int i = 0; i < kMaxVec; ++i) {
      const int c = threadIdx.x + i * kNormThreads;
      if (c < nvec) {
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = rstd * (gv[i][e] - xv[i][e] * dot);
        if (dres) {
          float r[8];
          load8(dres + off + c * 8, r);
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] += r[e];
        }
        store8(dx + off + c * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = threadIdx.x + i * kNormThreads;
    if (c < nvec) {
      float* dst = dw_partial + static_cast<size_t>(blockIdx.x) * D + c * 8;
      *reinterpret_cast<float4*>(dst) = make_float4(dw_acc[i][0], dw_acc[i][1], dw_acc[i][2], dw_acc[i][3]);
      *reinterpret_cast<float4*>(dst + 4) = make_float4(dw_acc[i][4], dw_acc[i][5], dw_acc[i][6], dw_acc[i][7]);
    }
  }
}

// dw[j] (+)= sum_p partial[p, j]; fixed summation order, so the result is run-to-run identical.
__global__ void colsum_partials_kernel(const float* __restrict__ partial, float* __restrict__ dw, int P, int D,
                                       int accumulate) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= D) return;
  float s = 0.f;
  for (int p = 0; p < P; ++p) s += partial[static_cast<size_t>(p) * D + j];
  dw[j] = accumulate ? dw[j] + s : s;
}

// A position outside the rotary table is an argument error: it is clamped (no out-of-range read) and
// reported through status bit 8.
__device__ __forceinline__ int checked_position(int pos, int table_rows, int* status, int lane) {
  if (pos >= 0 && pos < table_rows) return pos;
  if (lane == 0 && status != nullptr) atomicOr(status, 8);
  return pos < 0 ? 0 : table_rows - 1;
}

// One warp per (token, head). Heads [0, n_norm_q) use wq, heads [n_norm_q, n_rot) use wk for
// the optional per-head RMSNorm (wq == nullptr disables it); heads >= n_rot are copied.
// Rotation is the half-split form: (x1, x2) -> (x1 cos - x2 sin, x2 cos + x1 sin).
// `inverse` applies the transpose rotation (the backward of the forward rotation).
template <int H>
__global__ void __launch_bounds__(256)
qknorm_rope_fwd_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                       const int* __restrict__ positions, const float* __restrict__ cos_sin,
                       const __nv_bfloat16* __restrict__ wq, const __nv_bfloat16* __restrict__ wk,
                       float* __restrict__ rstd_out, long long T, int n_heads_total, int n_norm_q, int n_rot,
                       long long in_stride, long long out_stride, float eps, float w_offset, int inverse,
                       int table_rows, int* __restrict__ status, const long long* __restrict__ slots,
                       __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages) {
  constexpr int PER = H / 32;  // elements per lane (2, 4 or 8)
  const int lane = threadIdx.x & 31;
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long total = T * n_heads_total;
  if (gw >= total) return;
  const long long t = gw / n_heads_total;
  const int h = static_cast<int>(gw - t * n_heads_total);
  const __nv_bfloat16* src = in + t * in_stride + static_cast<long long>(h) * H + lane * PER;
  __nv_bfloat16* dst = out + t * out_stride + static_cast<long long>(h) * H + lane * PER;
  float v[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) v[e] = __bfloat162float(src[e]);
  if (h < n_rot) {
    if (wq != nullptr) {
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < PER; ++e) ss += v[e] * v[e];
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / H + eps);
      if (rstd_out && lane == 0) rstd_out[gw] = rstd;
      const __nv_bfloat16* w = (h < n_norm_q ? wq : wk) + lane * PER;
#pragma unroll
      for (int e = 0; e < PER; ++e) v[e] = v[e] * rstd * (__bfloat162float(w[e]) + w_offset);
      // the reference rounds the normalised value to the activation dtype before rotating
#pragma unroll
      for (int e = 0; e < PER; ++e) v[e] = __bfloat162float(__float2bfloat16_rn(v[e]));
    }
    const int pos = checked_position(positions[t], table_rows, status, lane);
    const float* cs = cos_sin + static_cast<long long>(pos) * H;  // [cos(H/2) | sin(H/2)]
#pragma unroll
    for (int e = 0; e < PER; ++e) {
      const float other = __shfl_xor_sync(0xffffffffu, v[e], 16);
      const int idx = (lane * PER + e) % (H / 2);
      const float c = cs[idx];
      float s = cs[H / 2 + idx];
      if (inverse) s = -s;
      v[e] = (lane < 16) ? (v[e] * c - other * s) : (v[e] * c + other * s);
    }
  }
#pragma unroll
  for (int e = 0; e < PER; ++e) dst[e] = __float2bfloat16_rn(v[e]);
  if (slots != nullptr && h >= n_norm_q) {
    // decode / prefill into a paged cache: the rotated key and the value also go to their page row
    const long long slot = slots[t];
    if (slot >= 0) {
      const int n_k = n_rot - n_norm_q;
      const bool is_k = h < n_rot;
      __nv_bfloat16* page = (is_k ? k_pages : v_pages) + slot * (static_cast<long long>(n_k) * H) +
                            static_cast<long long>(is_k ? h - n_norm_q : h - n_rot) * H + lane * PER;
#pragma unroll
      for (int e = 0; e < PER; ++e) page[e] = __float2bfloat16_rn(v[e]);
    }
  }
}

// Backward of qknorm_rope_fwd for the normalised heads: un-rotate dy, then RMSNorm backward
// per head. dw for the q and k norm weights is accumulated with atomics into dwq / dwk (fp32).
template <int H>
__global__ void __launch_bounds__(256)
qknorm_rope_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                       __nv_bfloat16* __restrict__ dx, const int* __restrict__ positions,
                       const float* __restrict__ cos_sin, const __nv_bfloat16* __restrict__ wq,
                       const __nv_bfloat16* __restrict__ wk, float* __restrict__ dwq, float* __restrict__ dwk,
                       long long T, int n_heads_total, int n_norm_q, int n_rot, long long x_stride,
                       long long dy_stride, long long dx_stride, float eps, float w_offset, int table_rows,
                       int* __restrict__ status) {
  constexpr int PER = H / 32;
  __shared__ float sdw[2][H];
  for (int i = threadIdx.x; i < 2 * H; i += blockDim.x) (&sdw[0][0])[i] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long total = T * n_heads_total;
  if (gw < total) {
    const long long t = gw / n_heads_total;
    const int h = static_cast<int>(gw - t * n_heads_total);
    const long long ho = static_cast<long long>(h) * H + lane * PER;
    float g[PER];
#pragma unroll
    for (int e = 0; e < PER; ++e) g[e] = __bfloat162float(dy[t * dy_stride + ho + e]);
    if (h < n_rot) {
      const int pos = checked_position(positions[t], table_rows, status, lane);
      const float* cs = cos_sin + static_cast<long long>(pos) * H;
#pragma unroll
      for (int e = 0; e < PER; ++e) {
        const float other = __shfl_xor_sync(0xffffffffu, g[e], 16);
        const int idx = (lane * PER + e) % (H / 2);
        const float c = cs[idx], s = -cs[H / 2 + idx];
        g[e] = (lane < 16) ? (g[e] * c - other * s) : (g[e] * c + other * s);
      }
      if (wq != nullptr) {
        float xv[PER];
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < PER; ++e) {
          xv[e] = __bfloat162float(x[t * x_stride + ho + e]);
          ss += xv[e] * xv[e];
        }
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / H + eps);
        const bool is_q = h < n_norm_q;
        const __nv_bfloat16* w = (is_q ? wq : wk) + lane * PER;
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < PER; ++e) {
          const float xh = xv[e] * rstd;
          atomicAdd(&sdw[is_q ? 0 : 1][lane * PER + e], g[e] * xh);
          g[e] *= (__bfloat162float(w[e]) + w_offset);
          dot += g[e] * xh;
          xv[e] = xh;
        }
        dot = warp_sum(dot) / H;
#pragma unroll
        for (int e = 0; e < PER; ++e) g[e] = rstd * (g[e] - xv[e] * dot);
      }
    }
#pragma unroll
    for (int e = 0; e < PER; ++e) dx[t * dx_stride + ho + e] = __float2bfloat16_rn(g[e]);
  }
  if (wq != nullptr) {
    __syncthreads();
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      if (sdw[0][i] != 0.f) atomicAdd(dwq + i, sdw[0][i]);
      if (sdw[1][i] != 0.f) atomicAdd(dwk + i, sdw[1][i]);
    }
  }
}

}  // namespace

extern "C" int tx_rmsnorm_fwd(const void* x, const void* res, const void* w, void* y, void* sum_out,
                              float* rstd, int T, int D, float eps, float w_offset, cudaStream_t stream) {
  if (D % 8 != 0 || D > kNormThreads * 8 * kMaxVec) return 1;
  if (T <= 0) return 0;
  const int cap = txh::sm_count() * 8;
  const int grid = T < cap ? T : cap;
  rmsnorm_fwd_kernel<<<grid, kNormThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(res),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y), static_cast<__nv_bfloat16*>(sum_out),
      rstd, T, D, eps, w_offset);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// Number of partial rows the backward kernel writes; the caller allocates
// dw_partial as [tx_rmsnorm_bwd_partials(T), D] fp32.
extern "C" int tx_rmsnorm_bwd_partials(int T) {
  int cap = txh::sm_count() * 2;
  if (cap > 296) cap = 296;      // the library-owned scratch of tx_rmsnorm_bwd_static holds 296 rows
  return T < cap ? (T > 0 ? T : 1) : cap;
}

extern "C" int tx_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, const void* dres,
                              void* dx, float* dw_partial, float* dw, int dw_accumulate, int T, int D, float eps,
                              float w_offset, cudaStream_t stream) {
  if (D % 8 != 0 || D > kNormThreads * 8 * kMaxVec) return 1;
  if (T <= 0) return 0;
  const int grid = tx_rmsnorm_bwd_partials(T);
  rmsnorm_bwd_kernel<<<grid, kNormThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(dy), rstd, static_cast<const __nv_bfloat16*>(dres),
      static_cast<__nv_bfloat16*>(dx), dw_partial, T, D, eps, w_offset);
  if (dw) colsum_partials_kernel<<<(D + 255) / 256, 256, 0, stream>>>(dw_partial, dw, grid, D, dw_accumulate);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

#define TX_DISPATCH_H(H, ...)                      \
  switch (H) {                                     \
    case 64: { constexpr int kH = 64; __VA_ARGS__; break; }   \
    case 128: { constexpr int kH = 128; __VA_ARGS__; break; } \
    case 256: { constexpr int kH = 256; __VA_ARGS__; break; } \
    default: return 1;                             \
  }

extern "C" int tx_qknorm_rope_fwd(const void* in, void* out, const int* positions, const float* cos_sin,
                                  const void* wq, const void* wk, float* rstd, long long T, int n_heads_total,
                                  int n_norm_q, int n_rot, int H, long long in_stride, long long out_stride,
                                  float eps, float w_offset, int inverse, int table_rows, int* status,
                                  const long long* slots, void* k_pages, void* v_pages, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (table_rows <= 0) return 1;
  if (slots != nullptr && (!k_pages || !v_pages || n_heads_total - n_rot != n_rot - n_norm_q)) return 1;
  const long long warps = T * n_heads_total;
  const int blocks = static_cast<int>((warps + 7) / 8);
  TX_DISPATCH_H(H, (qknorm_rope_fwd_kernel<kH><<<blocks, 256, 0, stream>>>(
                       static_cast<const __nv_bfloat16*>(in), static_cast<__nv_bfloat16*>(out), positions,
                       cos_sin, static_cast<const __nv_bfloat16*>(wq), static_cast<const __nv_bfloat16*>(wk),
                       rstd, T, n_heads_total, n_norm_q, n_rot, in_stride, out_stride, eps, w_offset, inverse,
                       table_rows, status, slots, static_cast<__nv_bfloat16*>(k_pages),
                       static_cast<__nv_bfloat16*>(v_pages))));
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

extern "C" int tx_qknorm_rope_bwd(const void* x, const void* dy, void* dx, const int* positions,
                                  const float* cos_sin, const void* wq, const void* wk, float* dwq, float* dwk,
                                  long long T, int n_heads_total, int n_norm_q, int n_rot, int H,
                                  long long x_stride, long long dy_stride, long long dx_stride, float eps,
                                  float w_offset, int table_rows, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (table_rows <= 0) return 1;
  const long long warps = T * n_heads_total;
  const int blocks = static_cast<int>((warps + 7) / 8);
  TX_DISPATCH_H(H, (qknorm_rope_bwd_kernel<kH><<<blocks, 256, 0, stream>>>(
                       static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
                       static_cast<__nv_bfloat16*>(dx), positions, cos_sin, static_cast<const __nv_bfloat16*>(wq),
                       static_cast<const __nv_bfloat16*>(wk), dwq, dwk, T, n_heads_total, n_norm_q, n_rot,
                       x_stride, dy_stride, dx_stride, eps, w_offset, table_rows, status)));
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// ---- RMSNorm backward with library-owned scratch (contract in norm_static.h) -----------------
#include <mutex>

#include "norm_static.h"

namespace {
constexpr int kStaticMaxD = 4096;
constexpr int kStaticMaxPartials = 148 * 2;   // upper bound of tx_rmsnorm_bwd_partials()
constexpr int kStaticMaxDevices = 64;
// One instance per device that loads this module. In host code the name below is only a
// handle for the symbol look-up, never a device address.
static __device__ __align__(256) float g_static_dw_partial[kStaticMaxPartials * kStaticMaxD];
float* g_static_dw_ptr[kStaticMaxDevices] = {};
std::mutex g_static_mu;

// Device address of the scratch on the current device; looked up once per device.
int static_scratch(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kStaticMaxDevices) return TX_STATIC_ERR_DEVICE;
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (g_static_dw_ptr[dev] == nullptr) {
    float* p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_dw_partial) != cudaSuccess || p == nullptr) {
      (void)cudaGetLastError();
      return TX_STATIC_ERR_SYMBOL;
    }
    g_static_dw_ptr[dev] = p;
  }
  *out = g_static_dw_ptr[dev];
  return TX_STATIC_OK;
}
}  // namespace

extern "C" int tx_rmsnorm_bwd_static_max_d(void) { return kStaticMaxD; }

extern "C" const char* tx_rmsnorm_bwd_static_strerror(int code) {
  switch (code) {
    case TX_STATIC_OK: return "ok";
    case TX_STATIC_ERR_BAD_SHAPE: return "tx_rmsnorm_bwd_static: D must be a multiple of 8 and T >= 0";
    case TX_STATIC_ERR_TOO_LARGE:
      return "tx_rmsnorm_bwd_static: D exceeds the built-in scratch (max 4096); use tx_rmsnorm_bwd with "
             "caller-provided scratch";
    case TX_STATIC_ERR_DEVICE: return "tx_rmsnorm_bwd_static: no current CUDA device, or its ordinal is >= 64";
    case TX_STATIC_ERR_SYMBOL: return "tx_rmsnorm_bwd_static: address look-up of the scratch array failed";
    case TX_STATIC_ERR_LAUNCH: return "tx_rmsnorm_bwd_static: kernel launch failed";
    default: return "tx_rmsnorm_bwd_static: unknown code";
  }
}

extern "C" int tx_rmsnorm_bwd_static(const void* x, const void* w, const void* dy, const float* rstd,
                                     const void* dres, void* dx, float* dw, int dw_accumulate, int T, int D,
                                     float eps, float w_offset, cudaStream_t stream) {
  if (D <= 0 || D % 8 != 0 || T < 0) return TX_STATIC_ERR_BAD_SHAPE;
  if (D > kStaticMaxD) return TX_STATIC_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = static_scratch(&scratch);   // also on T == 0, so that a start-up call does the set-up
  if (rc != TX_STATIC_OK) return rc;
  if (T == 0) return TX_STATIC_OK;
  const int grid = tx_rmsnorm_bwd_partials(T);   // <= kStaticMaxPartials rows of D <= kStaticMaxD floats
  rmsnorm_bwd_kernel<<<grid, kNormThreads, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(dy), rstd, static_cast<const __nv_bfloat16*>(dres),
      static_cast<__nv_bfloat16*>(dx), scratch, T, D, eps, w_offset);
  if (dw) colsum_partials_kernel<<<(D + 255) / 256, 256, 0, stream>>>(scratch, dw, grid, D, dw_accumulate);
  return cudaGetLastError() == cudaSuccess ? TX_STATIC_OK : TX_STATIC_ERR_LAUNCH;
}
