// Rollout-side kernels: KV-cache page write, paged decode attention (split-KV, GQA) and token
// sampling. All are bandwidth-bound; none uses tensor cores.
//
// Cache layout: k_pages / v_pages [num_pages, page_size, Kh, H] bf16. A sequence owns a list of
// pages (its row of `block_tables`); token t of the sequence lives in page block_tables[t / page]
// at row t % page. `slots[i] = page * page_size + row` addresses one token row directly.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "tx_host.h"

namespace {

// ------------------------------------------------------------------------------------------------
// KV page write: k_new/v_new [T, Kh*H] (row stride ld) -> pages at slots[T]. slot < 0 skips a row.
// ------------------------------------------------------------------------------------------------
__global__ void kv_page_write_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                     long long ldk, long long ldv, const long long* __restrict__ slots,
                                     __nv_bfloat16* __restrict__ k_pages, __nv_bfloat16* __restrict__ v_pages,
                                     int T, int row_elems) {
  const int vec_per_row = row_elems / 8;
  const long long total = static_cast<long long>(T) * vec_per_row;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / vec_per_row), c = static_cast<int>(i % vec_per_row);
    const long long slot = slots[t];
    if (slot < 0) continue;
    const uint4 kv = *reinterpret_cast<const uint4*>(k_new + t * ldk + c * 8);
    const uint4 vv = *reinterpret_cast<const uint4*>(v_new + t * ldv + c * 8);
    *reinterpret_cast<uint4*>(k_pages + slot * row_elems + c * 8) = kv;
    *reinterpret_cast<uint4*>(v_pages + slot * row_elems + c * 8) = vv;
  }
}

// ------------------------------------------------------------------------------------------------
// Paged decode attention. Grid (split, kv head, sequence); 4 warps per CTA. H/8 lanes own one key
// (8 contiguous dims each), so a warp handles 32/(H/8) keys per iteration and keeps, per lane
// group, an online-softmax state for each of the G = N/Kh query heads of the group. Lane groups,
// warps and splits are merged at the end (splits through a workspace and a second kernel).
// ------------------------------------------------------------------------------------------------
constexpr int kMaxG = 8;
constexpr int kDecWarps = 4;

template <int H, int G>
__global__ void __launch_bounds__(kDecWarps * 32)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, long long ldq, const __nv_bfloat16* __restrict__ k_pages,
                    const __nv_bfloat16* __restrict__ v_pages, const int* __restrict__ block_tables,
                    int max_blocks, const int* __restrict__ seq_lens, int page_size, int Kh, float scale_log2,
                    int num_splits, float* __restrict__ ws_o, float* __restrict__ ws_ml,
                    __nv_bfloat16* __restrict__ out, long long ldo) {
  constexpr int LPK = H / 8;            // lanes per key
  constexpr int KPW = 32 / LPK;         // keys per warp iteration
  // lets a programmatically launched successor (the output-projection GEMM) prefetch its weights meanwhile
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPK, dl = lane % LPK;
  const int len = seq_lens[b];
  const int N = Kh * G;
  // keys of this split: [lo, hi)
  const int per = (len + num_splits - 1) / num_splits;
  const int lo = split * per, hi = min(len, lo + per);

  float qv[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 u = *reinterpret_cast<const uint4*>(q + b * ldq + (kvh * G + g) * H + dl * 8);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h2[i]);
      qv[g][2 * i] = f.x * scale_log2;
      qv[g][2 * i + 1] = f.y * scale_log2;
    }
  }
  float m[G], l[G], o[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) o[g][i] = 0.f;
  }
  const int* bt = block_tables + static_cast<long long>(b) * max_blocks;
  const long long row_elems = static_cast<long long>(Kh) * H;
  for (int t0 = lo + warp * KPW; t0 < hi; t0 += kDecWarps * KPW) {
    const int t = t0 + sub;
    const bool valid = t < hi;
    float kf[8], vf[8];
    if (valid) {
      const long long row = (static_cast<long long>(bt[t / page_size]) * page_size + t % page_size) * row_elems +
                            kvh * H + dl * 8;
      const uint4 ku = *reinterpret_cast<const uint4*>(k_pages + row);
      const uint4 vu = *reinterpret_cast<const uint4*>(v_pages + row);
      const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&ku);
      const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vu);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 a = __bfloat1622float2(k2[i]), c = __bfloat1622float2(v2[i]);
        kf[2 * i] = a.x; kf[2 * i + 1] = a.y;
        vf[2 * i] = c.x; vf[2 * i + 1] = c.y;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) kf[i] = vf[i] = 0.f;
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s += qv[g][i] * kf[i];
#pragma unroll
      for (int off = LPK / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
      if (valid) {
        const float mn = fmaxf(m[g], s);
        const float alpha = exp2f(m[g] - mn), p = exp2f(s - mn);
        m[g] = mn;
        l[g] = l[g] * alpha + p;
#pragma unroll
        for (int i = 0; i < 8; ++i) o[g][i] = o[g][i] * alpha + p * vf[i];
      }
    }
  }
  // merge the lane groups of a warp (butterfly over the `sub` bits)
#pragma unroll
  for (int off = LPK; off < 32; off <<= 1) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[g], off);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[g], off);
      const float mn = fmaxf(m[g], m2);
      const float a1 = (m[g] == -INFINITY) ? 0.f : exp2f(m[g] - mn);
      const float a2 = (m2 == -INFINITY) ? 0.f : exp2f(m2 - mn);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float o2 = __shfl_xor_sync(0xffffffffu, o[g][i], off);
        o[g][i] = o[g][i] * a1 + o2 * a2;
      }
      l[g] = l[g] * a1 + l2 * a2;
      m[g] = mn;
    }
  }
  // merge the warps through shared memory
  __shared__ float sh_o[kDecWarps][G][H];
  __shared__ float sh_m[kDecWarps][G], sh_l[kDecWarps][G];
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
      for (int i = 0; i < 8; ++i) sh_o[warp][g][dl * 8 + i] = o[g][i];
      if (dl == 0) { sh_m[warp][g] = m[g]; sh_l[warp][g] = l[g]; }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * H; idx += kDecWarps * 32) {
    const int g = idx / H, d = idx % H;
    float mn = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) mn = fmaxf(mn, sh_m[w][g]);
    float acc = 0.f, ls = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float a = (sh_m[w][g] == -INFINITY) ? 0.f : exp2f(sh_m[w][g] - mn);
      acc += sh_o[w][g][d] * a;
      ls += sh_l[w][g] * a;
    }
    const int head = kvh * G + g;
    if (num_splits == 1) {
      out[b * ldo + head * H + d] = __float2bfloat16_rn(ls > 0.f ? acc / ls : 0.f);
    } else {
      const long long base = (static_cast<long long>(b) * N + head) * num_splits + split;
      ws_o[base * H + d] = acc;
      if (d == 0) { ws_ml[base * 2] = mn; ws_ml[base * 2 + 1] = ls; }
    }
  }
}

template <int H>
__global__ void paged_decode_combine_kernel(const float* __restrict__ ws_o, const float* __restrict__ ws_ml,
                                            int num_splits, __nv_bfloat16* __restrict__ out, long long ldo, int N) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int head = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const long long base = (static_cast<long long>(b) * N + head) * num_splits;
  float mn = -INFINITY;
  for (int s = 0; s < num_splits; ++s) mn = fmaxf(mn, ws_ml[(base + s) * 2]);
  float acc = 0.f, ls = 0.f;
  for (int s = 0; s < num_splits; ++s) {
    const float ms = ws_ml[(base + s) * 2];
    const float a = (ms == -INFINITY) ? 0.f : exp2f(ms - mn);
    acc += ws_o[(base + s) * H + d] * a;
    ls += ws_ml[(base + s) * 2 + 1] * a;
  }
  out[b * ldo + head * H + d] = __float2bfloat16_rn(ls > 0.f ? acc / ls : 0.f);
}

}  // namespace

// ------------------------------------------------------------------------------------------------
// Sampling: greedy, or exact categorical sampling at a temperature by the Gumbel-max trick
// (argmax_i z_i + g_i with g_i = -log(-log u_i)), in one pass over the row. u comes from
// Philox-4x32-10 keyed by (seed, step) with counter (row, i / 4), so a draw depends only on
// (seed, step, row, i) and not on batch composition or launch geometry. Also returns the
// log-probability of the chosen token under softmax(z), z = logits / temperature.
// ------------------------------------------------------------------------------------------------
namespace {

__device__ __forceinline__ void philox_round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c[0];
  const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c[2];
  const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0;
  const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
  c[1] = static_cast<uint32_t>(p1);
  c[3] = static_cast<uint32_t>(p0);
  c[0] = n0;
  c[2] = n2;
}

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

__device__ __forceinline__ float gumbel_from_bits(uint32_t bits) {
  const float u = (static_cast<float>(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);   // (0, 1)
  return -__logf(-__logf(u));
}

template <typename T>
__device__ __forceinline__ float load_logit(const T* p, long long i);
template <>
__device__ __forceinline__ float load_logit<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float load_logit<__nv_bfloat16>(const __nv_bfloat16* p, long long i) {
  return __bfloat162float(p[i]);
}

constexpr int kSampleThreads = 1024;   // one CTA per row: the row (up to ~150k logits) is scanned once, 4 logits per thread and step

template <typename T>
__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const T* __restrict__ logits, long long ld, int V, float inv_temp, int greedy,
              unsigned long long seed, const long long* __restrict__ step_ptr, long long step_add,
              const int* __restrict__ forbidden, int n_forbidden, long long* __restrict__ tokens,
              float* __restrict__ logprobs) {
  const int row = blockIdx.x;
  const T* x = logits + static_cast<long long>(row) * ld;
  const unsigned long long step = static_cast<unsigned long long>((step_ptr ? *step_ptr : 0) + step_add);
  const uint32_t k0 = static_cast<uint32_t>(seed) ^ static_cast<uint32_t>(step * 0x9E3779B97F4A7C15ull >> 32);
  const uint32_t k1 = static_cast<uint32_t>(seed >> 32) ^ static_cast<uint32_t>(step);
  float m = -INFINITY, se = 0.f, best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i4 = threadIdx.x * 4; i4 < V; i4 += kSampleThreads * 4) {
    uint32_t c[4] = {static_cast<uint32_t>(i4 >> 2), static_cast<uint32_t>(row), 0x5eedu, 0u};
    if (!greedy) philox4x32_10(c, k0, k1);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = i4 + e;
      if (i >= V) break;
      float z = load_logit<T>(x, i) * inv_temp;
      for (int f = 0; f < n_forbidden; ++f)
        if (forbidden[f] == i) z = -INFINITY;
      if (z > m) {
        se = se * __expf(m - z) + 1.f;
        m = z;
      } else if (z > -INFINITY) {
        se += __expf(z - m);
      }
      const float key = greedy ? z : z + gumbel_from_bits(c[e]);
      if (key > best || (key == best && i < best_i)) {
        best = key;
        best_i = i;
      }
    }
  }
  __shared__ float sm[kSampleThreads], ss[kSampleThreads], sb[kSampleThreads];
  __shared__ int si[kSampleThreads];
  sm[threadIdx.x] = m; ss[threadIdx.x] = se; sb[threadIdx.x] = best; si[threadIdx.x] = best_i;
  __syncthreads();
  for (int o = kSampleThreads / 2; o > 0; o >>= 1) {
    if (threadIdx.x < o) {
      const float m1 = sm[threadIdx.x], m2 = sm[threadIdx.x + o];
      const float mn = fmaxf(m1, m2);
      const float a1 = (m1 == -INFINITY) ? 0.f : __expf(m1 - mn), a2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
      ss[threadIdx.x] = ss[threadIdx.x] * a1 + ss[threadIdx.x + o] * a2;
      sm[threadIdx.x] = mn;
      const float b2 = sb[threadIdx.x + o];
      const int i2 = si[threadIdx.x + o];
      if (b2 > sb[threadIdx.x] || (b2 == sb[threadIdx.x] && i2 < si[threadIdx.x])) {
        sb[threadIdx.x] = b2;
        si[threadIdx.x] = i2;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const int tok = si[0] < V ? si[0] : 0;
    tokens[row] = tok;
    if (logprobs) logprobs[row] = load_logit<T>(x, tok) * inv_temp - (sm[0] + __logf(ss[0]));
  }
}

template <int H>
int launch_decode(int G, dim3 grid, cudaStream_t s, const __nv_bfloat16* q, long long ldq, const __nv_bfloat16* kp,
                  const __nv_bfloat16* vp, const int* bt, int max_blocks, const int* lens, int page, int Kh,
                  float scale_log2, int splits, float* ws_o, float* ws_ml, __nv_bfloat16* out, long long ldo) {
#define TX_DEC_CASE(GG)                                                                                      \
  case GG:                                                                                                   \
    paged_decode_kernel<H, GG><<<grid, kDecWarps * 32, 0, s>>>(q, ldq, kp, vp, bt, max_blocks, lens, page, Kh, \
                                                               scale_log2, splits, ws_o, ws_ml, out, ldo);   \
    break;
  switch (G) {
    TX_DEC_CASE(1) TX_DEC_CASE(2) TX_DEC_CASE(3) TX_DEC_CASE(4) TX_DEC_CASE(5) TX_DEC_CASE(6) TX_DEC_CASE(7)
    TX_DEC_CASE(8)
    default: return 1;
  }
#undef TX_DEC_CASE
  if (splits > 1) {
    dim3 g2(Kh * G, grid.z);
    paged_decode_combine_kernel<H><<<g2, H, 0, s>>>(ws_o, ws_ml, splits, out, ldo, Kh * G);
  }
  return 0;
}

}  // namespace

extern "C" int tx_kv_page_write(const void* k_new, const void* v_new, long long ldk, long long ldv,
                                const long long* slots, void* k_pages, void* v_pages, int T, int Kh, int H,
                                cudaStream_t s) {
  const int row_elems = Kh * H;
  if (T <= 0) return 0;
  if (row_elems % 8 != 0 || ldk % 8 != 0 || ldv % 8 != 0) return 1;
  const long long total = static_cast<long long>(T) * (row_elems / 8);
  const long long cap = static_cast<long long>(txh::sm_count()) * 16;
  const int blocks = static_cast<int>(total / 256 + 1 < cap ? total / 256 + 1 : cap);
  kv_page_write_kernel<<<blocks, 256, 0, s>>>(static_cast<const __nv_bfloat16*>(k_new),
                                              static_cast<const __nv_bfloat16*>(v_new), ldk, ldv, slots,
                                              static_cast<__nv_bfloat16*>(k_pages),
                                              static_cast<__nv_bfloat16*>(v_pages), T, row_elems);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// Merges the per-split partial results (ws_o unnormalised fp32 sums relative to ws_ml's max, ws_ml = (max in
// log2 units, sum)) into out [B, N*H] bf16. Used by the tensor-core decode kernel, which writes the same layout.
extern "C" int tx_paged_decode_combine(const float* ws_o, const float* ws_ml, int num_splits, void* out,
                                       long long ldo, int B, int N, int H, cudaStream_t s) {
  if (B <= 0) return 0;
  if (!ws_o || !ws_ml || num_splits < 1) return 1;
  dim3 g2(N, B);
  auto* op = static_cast<__nv_bfloat16*>(out);
  switch (H) {
    case 64: paged_decode_combine_kernel<64><<<g2, 64, 0, s>>>(ws_o, ws_ml, num_splits, op, ldo, N); break;
    case 128: paged_decode_combine_kernel<128><<<g2, 128, 0, s>>>(ws_o, ws_ml, num_splits, op, ldo, N); break;
    case 256: paged_decode_combine_kernel<256><<<g2, 256, 0, s>>>(ws_o, ws_ml, num_splits, op, ldo, N); break;
    default: return 1;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// Workspace for num_splits > 1: ws_o [B*N*splits*H] floats, ws_ml [B*N*splits*2] floats.
extern "C" int tx_paged_decode_attn(const void* q, long long ldq, const void* k_pages, const void* v_pages,
                                    const int* block_tables, int max_blocks, const int* seq_lens, int B, int N, int Kh,
                                    int H, int page_size, float scale, int num_splits, float* ws_o, float* ws_ml,
                                    void* out, long long ldo, cudaStream_t s) {
  if (B <= 0) return 0;
  if (Kh <= 0 || N % Kh != 0 || N / Kh > kMaxG || num_splits < 1 || (num_splits > 1 && (!ws_o || !ws_ml))) return 1;
  const int G = N / Kh;
  dim3 grid(num_splits, Kh, B);
  const float sl2 = scale * 1.4426950408889634f;
  const auto* qp = static_cast<const __nv_bfloat16*>(q);
  const auto* kp = static_cast<const __nv_bfloat16*>(k_pages);
  const auto* vp = static_cast<const __nv_bfloat16*>(v_pages);
  auto* op = static_cast<__nv_bfloat16*>(out);
  int rc;
  switch (H) {
    case 64: rc = launch_decode<64>(G, grid, s, qp, ldq, kp, vp, block_tables, max_blocks, seq_lens, page_size, Kh, sl2, num_splits, ws_o, ws_ml, op, ldo); break;
    case 128: rc = launch_decode<128>(G, grid, s, qp, ldq, kp, vp, block_tables, max_blocks, seq_lens, page_size, Kh, sl2, num_splits, ws_o, ws_ml, op, ldo); break;
    case 256: rc = launch_decode<256>(G, grid, s, qp, ldq, kp, vp, block_tables, max_blocks, seq_lens, page_size, Kh, sl2, num_splits, ws_o, ws_ml, op, ldo); break;
    default: return 1;
  }
  if (rc) return rc;
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// logits [B, V] fp32 (is_bf16 = 0) or bf16; tokens int64 [B]; logprobs fp32 [B] or null. The draw of
// row r uses step = *step_ptr + step_add (step_ptr may be null).
extern "C" int tx_sample(const void* logits, int is_bf16, long long ld, int B, int V, float temperature, int greedy,
                         unsigned long long seed, const long long* step_ptr, long long step_add,
                         const int* forbidden, int n_forbidden, long long* tokens, float* logprobs,
                         cudaStream_t s) {
  if (B <= 0) return 0;
  if (V <= 0 || (!greedy && !(temperature > 0.f))) return 1;
  const float inv = greedy ? 1.f : 1.f / temperature;
  if (is_bf16)
    sample_kernel<__nv_bfloat16><<<B, kSampleThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), ld, V, inv,
                                                              greedy, seed, step_ptr, step_add, forbidden,
                                                              n_forbidden, tokens, logprobs);
  else
    sample_kernel<float><<<B, kSampleThreads, 0, s>>>(static_cast<const float*>(logits), ld, V, inv, greedy, seed,
                                                      step_ptr, step_add, forbidden, n_forbidden, tokens, logprobs);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}
