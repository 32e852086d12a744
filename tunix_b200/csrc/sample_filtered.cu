// Top-k / top-p (nucleus) sampling in one launch, one CTA per row, nothing but shared memory as scratch.
//
// Semantics (tunix/generate/sampler.py:105-161): z = logits / temperature; the candidates are the k
// largest z; among them, in descending order, a token stays while the probability mass (softmax within
// the candidates) of the tokens strictly before it is <= top_p; the draw is categorical over the
// survivors; the reported log-prob is that of the drawn token under the FULL softmax(z).
//
// No sort. With d = max(z) - z >= 0, every token is given a three-level bin address (1024 bins per
// level over d in [0, 32): resolution 2^-25, finer than an fp32 logit near its maximum). "The k largest"
// and "mass before me <= p * Z" are both prefixes in that address order, so each is found by three
// histogram passes over the row (level by level into the boundary bin), counts as integers and
// masses as 40-bit fixed point, so the sums - and with them the survivor set - do not depend on the
// order of the shared-memory atomics: a row's result depends only on (seed, step, row, logits).
// Tokens sharing the last-level boundary bin are kept together (ties); tokens with d >= 32 (probability
// below e^-32 of the maximum) are never drawn while a filter is active. The final pass is the same
// Gumbel-max draw, with the same Philox counters, as the unfiltered kernel in decode.cu.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

namespace {

constexpr int kThreads = 512;
constexpr int kBins = 1024;          // 2 bins per thread in the scans
constexpr float kRange = 32.f;
constexpr float kMassScale = 1099511627776.f;   // 2^40

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
  const float u = (static_cast<float>(bits >> 8) + 0.5f) * (1.0f / 16777216.0f);
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

// Bin address of a distance d in [0, kRange): packed b1 << 20 | b2 << 10 | b3, increasing with d.
__device__ __forceinline__ uint32_t address_of(float d) {
  float t = d * (kBins / kRange);
  int b1 = static_cast<int>(t);
  b1 = b1 > kBins - 1 ? kBins - 1 : b1;
  t = (t - b1) * kBins;
  int b2 = static_cast<int>(t);
  b2 = b2 > kBins - 1 ? kBins - 1 : (b2 < 0 ? 0 : b2);
  t = (t - b2) * kBins;
  int b3 = static_cast<int>(t);
  b3 = b3 > kBins - 1 ? kBins - 1 : (b3 < 0 ? 0 : b3);
  return (static_cast<uint32_t>(b1) << 20) | (static_cast<uint32_t>(b2) << 10) | static_cast<uint32_t>(b3);
}

struct Shared {
  unsigned int count[kBins];
  unsigned long long mass[kBins];
  unsigned int warp_c[kThreads / 32];
  unsigned long long warp_m[kThreads / 32];
  float red_m[kThreads / 32], red_s[kThreads / 32], red_b[kThreads / 32];
  int red_i[kThreads / 32];
  int pick;                       // boundary bin chosen by the scan
  unsigned int before_c;          // count / mass in the bins before it (this level)
  unsigned long long before_m;
  unsigned int total_c;
  unsigned long long total_m;
};

// Exclusive prefix sums over the histogram: thread t owns bins 2t and 2t + 1. Returns through ec / em the
// exclusive prefix of bin 2t; totals land in sh.total_*.
__device__ __forceinline__ void scan_bins(Shared& sh, unsigned int& ec, unsigned long long& em) {
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const unsigned int c = sh.count[2 * t] + sh.count[2 * t + 1];
  const unsigned long long m = sh.mass[2 * t] + sh.mass[2 * t + 1];
  unsigned int ic = c;
  unsigned long long im = m;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned int vc = __shfl_up_sync(0xffffffffu, ic, o);
    const unsigned long long vm = __shfl_up_sync(0xffffffffu, im, o);
    if (lane >= o) { ic += vc; im += vm; }
  }
  if (lane == 31) { sh.warp_c[warp] = ic; sh.warp_m[warp] = im; }
  __syncthreads();
  unsigned int bc = 0;
  unsigned long long bm = 0;
  for (int w = 0; w < warp; ++w) { bc += sh.warp_c[w]; bm += sh.warp_m[w]; }
  if (t == kThreads - 1) { sh.total_c = bc + ic; sh.total_m = bm + im; }
  ec = bc + ic - c;
  em = bm + im - m;
  __syncthreads();
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
sample_filtered_kernel(const T* __restrict__ logits, long long ld, int V, float inv_temp, int top_k, float top_p,
                       unsigned long long seed, const long long* __restrict__ step_ptr, long long step_add,
                       const int* __restrict__ forbidden, int n_forbidden, long long* __restrict__ tokens,
                       float* __restrict__ logprobs) {
  __shared__ Shared sh;
  const int row = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const T* x = logits + static_cast<long long>(row) * ld;
  auto zval = [&](int i) -> float {
    float z = load_logit<T>(x, i) * inv_temp;
    for (int f = 0; f < n_forbidden; ++f)
      if (forbidden[f] == i) z = -INFINITY;
    return z;
  };

  // ---- pass 0: max and sum of exp over the whole row (fixed reduction order)
  float m = -INFINITY, se = 0.f;
  for (int i = t; i < V; i += kThreads) {
    const float z = zval(i);
    if (z > m) { se = se * __expf(m - z) + 1.f; m = z; }
    else if (z > -INFINITY) se += __expf(z - m);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, se, o);
    const float mn = fmaxf(m, m2);
    se = (m == -INFINITY ? 0.f : se * __expf(m - mn)) + (m2 == -INFINITY ? 0.f : s2 * __expf(m2 - mn));
    m = mn;
  }
  if (lane == 0) { sh.red_m[warp] = m; sh.red_s[warp] = se; }
  __syncthreads();
  {
    float mm = -INFINITY;
    for (int w = 0; w < kThreads / 32; ++w) mm = fmaxf(mm, sh.red_m[w]);
    float ss = 0.f;
    for (int w = 0; w < kThreads / 32; ++w)
      if (sh.red_m[w] > -INFINITY) ss += sh.red_s[w] * __expf(sh.red_m[w] - mm);
    m = mm;
    se = ss;
  }
  __syncthreads();

  // ---- boundaries: addresses <= bound_k are the k largest; addresses <= bound_p pass the nucleus test
  uint32_t bound_k = 0xffffffffu, bound_p = 0xffffffffu;
  unsigned long long z_k = 0;                 // mass of the top-k set (fixed point)
  const bool use_k = top_k > 0 && top_k < V;
  const bool use_p = top_p < 1.f;
  for (int phase = 0; phase < 2; ++phase) {
    if (phase == 0 && !use_k && !use_p) break;
    if (phase == 1 && !use_p) break;
    // phase 0 always runs when any filter is active: it also measures z_k (with no top-k: the mass in range)
    uint32_t prefix = 0;                      // chosen bins of the levels above, in address position
    unsigned int need = use_k ? static_cast<unsigned int>(top_k) : 0xffffffffu;
    unsigned long long acc_m = 0;             // mass before the boundary, over the levels so far
    const unsigned long long limit =
        phase == 1 ? static_cast<unsigned long long>(static_cast<double>(z_k) * static_cast<double>(top_p)) : 0;
    bool open = true;                          // false once the boundary is known to be "everything in range"
    for (int level = 0; level < 3 && open; ++level) {
      for (int b = t; b < kBins; b += kThreads) { sh.count[b] = 0; sh.mass[b] = 0; }
      __syncthreads();
      const int shift = 20 - 10 * level;
      const uint32_t upper_mask = level == 0 ? 0u : (0xffffffffu << (shift + 10)) & 0x3fffffffu;
      for (int i = t; i < V; i += kThreads) {
        const float d = m - zval(i);
        if (!(d < kRange)) continue;
        const uint32_t a = address_of(d);
        if ((a & upper_mask) != (prefix & upper_mask)) continue;
        if (phase == 1 && a > bound_k) continue;
        const int bin = (a >> shift) & (kBins - 1);
        atomicAdd(&sh.count[bin], 1u);
        atomicAdd(&sh.mass[bin], static_cast<unsigned long long>(__float2ull_rd(__expf(-d) * kMassScale)));
      }
      __syncthreads();
      unsigned int ec;
      unsigned long long em;
      scan_bins(sh, ec, em);
      if (t == 0) sh.pick = -1;
      __syncthreads();
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int bin = 2 * t + j;
        const unsigned int c_ex = ec + (j ? sh.count[2 * t] : 0u);
        const unsigned long long m_ex = em + (j ? sh.mass[2 * t] : 0ull);
        bool hit;
        if (phase == 0) {
          hit = c_ex < need && c_ex + sh.count[bin] >= need;      // the bin holding the need-th largest
        } else {
          const unsigned long long m_in = m_ex + sh.mass[bin];
          hit = acc_m + m_ex <= limit && (bin == kBins - 1 || acc_m + m_in > limit);   // last bin whose top passes
        }
        if (hit) { sh.pick = bin; sh.before_c = c_ex; sh.before_m = m_ex; }
      }
      __syncthreads();
      const int pick = sh.pick;
      if (pick < 0) {
        // fewer than `need` tokens in range (phase 0): everything in range is kept
        acc_m += sh.total_m;
        open = false;
        prefix = 0xffffffffu;
      } else {
        prefix |= static_cast<uint32_t>(pick) << shift;
        need -= sh.before_c;
        acc_m += sh.before_m;
        if (level == 2) acc_m += sh.mass[pick];       // the last-level boundary bin is kept whole
      }
      __syncthreads();
    }
    if (phase == 0) {
      bound_k = use_k ? prefix : 0xffffffffu;
      z_k = acc_m;
    } else {
      bound_p = prefix;
    }
  }
  const uint32_t bound = bound_k < bound_p ? bound_k : bound_p;

  // ---- final pass: Gumbel-max among the survivors (Philox counters as in the unfiltered kernel)
  const unsigned long long step = static_cast<unsigned long long>((step_ptr ? *step_ptr : 0) + step_add);
  const uint32_t k0 = static_cast<uint32_t>(seed) ^ static_cast<uint32_t>(step * 0x9E3779B97F4A7C15ull >> 32);
  const uint32_t k1 = static_cast<uint32_t>(seed >> 32) ^ static_cast<uint32_t>(step);
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i4 = t * 4; i4 < V; i4 += kThreads * 4) {
    uint32_t c[4] = {static_cast<uint32_t>(i4 >> 2), static_cast<uint32_t>(row), 0x5eedu, 0u};
    philox4x32_10(c, k0, k1);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = i4 + e;
      if (i >= V) break;
      const float z = zval(i);
      const float d = m - z;
      if (!(d < kRange) || address_of(d) > bound) continue;
      const float key = z + gumbel_from_bits(c[e]);
      if (key > best || (key == best && i < best_i)) { best = key; best_i = i; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float b2 = __shfl_xor_sync(0xffffffffu, best, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, best_i, o);
    if (b2 > best || (b2 == best && i2 < best_i)) { best = b2; best_i = i2; }
  }
  if (lane == 0) { sh.red_b[warp] = best; sh.red_i[warp] = best_i; }
  __syncthreads();
  if (t == 0) {
    for (int w = 1; w < kThreads / 32; ++w)
      if (sh.red_b[w] > best || (sh.red_b[w] == best && sh.red_i[w] < best_i)) { best = sh.red_b[w]; best_i = sh.red_i[w]; }
    const int tok = best_i < V ? best_i : 0;
    tokens[row] = tok;
    if (logprobs) logprobs[row] = zval(tok) - (m + __logf(se));
  }
}

}  // namespace

// Like tx_sample (decode.cu) with top_k (<= 0: off) and top_p (>= 1: off) applied before the draw.
extern "C" int tx_sample_filtered(const void* logits, int is_bf16, long long ld, int B, int V, float temperature,
                                  int top_k, float top_p, unsigned long long seed, const long long* step_ptr,
                                  long long step_add, const int* forbidden, int n_forbidden, long long* tokens,
                                  float* logprobs, cudaStream_t s) {
  if (B <= 0) return 0;
  if (V <= 0 || !(temperature > 0.f) || !(top_p > 0.f)) return 1;
  const float inv = 1.f / temperature;
  if (is_bf16)
    sample_filtered_kernel<__nv_bfloat16><<<B, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(logits), ld, V, inv,
                                                                 top_k, top_p, seed, step_ptr, step_add, forbidden,
                                                                 n_forbidden, tokens, logprobs);
  else
    sample_filtered_kernel<float><<<B, kThreads, 0, s>>>(static_cast<const float*>(logits), ld, V, inv, top_k, top_p,
                                                         seed, step_ptr, step_add, forbidden, n_forbidden, tokens,
                                                         logprobs);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}
