// Flash attention backward for head_dim 128 on tcgen05 tensor cores, as two kernels with a
// fixed reduction order (bitwise reproducible, no atomics):
//
//   flash_bwd_dkv_kernel  one CTA per (128 keys, kv head, batch). K and V stay in shared memory;
//       the CTA walks over every query head of the group and every 64-row query tile that can
//       see these keys and works on the transposed problem, so that keys are the M dimension
//       (TMEM lanes) of every product:
//         S^T  = K Q^T            dP^T = V dO^T                 (128 x 64, K = head dim)
//         P^T  = exp2(S^T*c - lse)   dS^T = P^T * (dP^T - delta)   (one thread per key row)
//         dV  += P^T dO           dK  += dS^T Q                 (128 x 128, K = 64 queries)
//       The Q and dO tiles serve as K-major B operands of the first pair and as MN-major B
//       operands of the second pair without being moved.
//   flash_bwd_dq_kernel   one CTA per (128 queries, head, batch), looping over 64-key tiles:
//         S = Q K^T, dP = dO V^T, dS = P * (dP - delta), dQ += dS K.
//
// delta[b,h,i] = sum_d dO[i,d] * O[i,d] comes from flash_bwd_delta_kernel. Roles inside a CTA
// are those of the forward kernel: warp 0 TMA producer, warp 1 MMA issuer; the elementwise work
// between the two product pairs has no row reduction (lse and delta are inputs), so it is split
// over 8 warps: warps 2..5 take columns 0..31 of their TMEM lanes, warps 6..9 columns 32..63.
// Every wait is bounded and reports through the status word.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "tx_host.h"
#include "tx_ptx.cuh"

namespace {
using namespace tx;

constexpr int kHD = 128;
constexpr int kThreads = 320;   // warp 0 producer, warp 1 MMA issuer, warps 2..9 elementwise (two per TMEM lane quarter)
constexpr float kLog2e = 1.4426950408889634f;

struct BwdParams {
  const float* lse;     // [B, N, Lq] natural log
  const float* delta;   // [B, N, Lq]
  __nv_bfloat16* out0;  // dkv: dK, dq: dQ
  __nv_bfloat16* out1;  // dkv: dV
  long long ld0, ld1;
  int B, N, Kh, Lq, Lk, causal;
  float scale, scale_log2;
  int* status;
  // Packed sequences (optional, Lq == Lk): first / last token index of each token's segment, [B, Lq].
  // Key k is visible to query q when seg_lo[q] <= k <= (causal ? q : seg_hi[q]).
  const int* seg_lo;
  const int* seg_hi;
};

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Writes 64 bf16 (as 32 packed words) to row r of a K-major 128-byte-swizzled [rows x 64] tile.
__device__ __forceinline__ void store_row_sw128(uint8_t* tile, int r, const uint32_t (&pk)[32]) {
  uint8_t* row = tile + r * 128;
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<uint4*>(row + ((c ^ (r & 7)) << 4)) =
        make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
}

// Half a row: 32 bf16 (16 packed words) into 16-byte chunks [4 ch, 4 ch + 4) of row r.
__device__ __forceinline__ void store_half_row_sw128(uint8_t* tile, int r, int ch, const uint32_t (&pk)[16]) {
  uint8_t* row = tile + r * 128;
#pragma unroll
  for (int c = 0; c < 4; ++c)
    *reinterpret_cast<uint4*>(row + (((ch * 4 + c) ^ (r & 7)) << 4)) =
        make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
}

// TMEM accumulator columns [c0, c1) of [128 lanes x 128 cols] -> bf16 rows in global memory, scaled.
__device__ __forceinline__ void store_acc_rows(uint32_t taddr, __nv_bfloat16* row_ptr, bool in_range, float mul,
                                               bool have_data, int c0 = 0, int c1 = kHD) {
#pragma unroll 1
  for (int c = c0; c < c1; c += 32) {
    uint32_t t[32];
    if (have_data) {
      tmem_ld_32x32b_x32(taddr + c, t);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) t[i] = 0u;
    }
    if (in_range) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 v;
        v.x = pack2(__uint_as_float(t[i]) * mul, __uint_as_float(t[i + 1]) * mul);
        v.y = pack2(__uint_as_float(t[i + 2]) * mul, __uint_as_float(t[i + 3]) * mul);
        v.z = pack2(__uint_as_float(t[i + 4]) * mul, __uint_as_float(t[i + 5]) * mul);
        v.w = pack2(__uint_as_float(t[i + 6]) * mul, __uint_as_float(t[i + 7]) * mul);
        *reinterpret_cast<uint4*>(row_ptr + c + i) = v;
      }
    }
  }
}

// delta = rowsum(dO * O); one warp per (token, head).
__global__ void flash_bwd_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                       float* __restrict__ delta, long long ldo, long long lddo, int B, int N,
                                       int L) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (w >= static_cast<long long>(B) * L * N) return;
  const int h = static_cast<int>(w % N);
  const long long tok = w / N;
  const uint2 a = *reinterpret_cast<const uint2*>(o + tok * ldo + h * kHD + lane * 4);
  const uint2 g = *reinterpret_cast<const uint2*>(d_o + tok * lddo + h * kHD + lane * 4);
  const float2 a0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.x));
  const float2 a1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a.y));
  const float2 g0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g.x));
  const float2 g1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&g.y));
  float s = a0.x * g0.x + a0.y * g0.y + a1.x * g1.x + a1.y * g1.y;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    const long long b = tok / L, i = tok % L;
    delta[(b * N + h) * L + i] = s;
  }
}

// ------------------------------------------------------------------------------------------------
// dK / dV
// ------------------------------------------------------------------------------------------------
namespace dkv {
constexpr int kKeys = 128, kQT = 64;
constexpr int kKBytes = kKeys * kHD * 2;       // 32 KiB, two [128 x 64] sub-tiles
constexpr int kQBytes = kQT * kHD * 2;         // 16 KiB, two [64 x 64] sub-tiles
constexpr int kPBytes = kKeys * kQT * 2;       // 16 KiB
constexpr int kQStages = 3;                    // Q / dO ring: a tile is requested two iterations ahead of its use
constexpr int kTileBytes = 2 * kKBytes + 2 * kQStages * kQBytes + 2 * kPBytes;   // 196608
constexpr int kVecBytes = 4 * 2 * kQT * 4;     // lse, delta, segment lo and hi; two buffers each
constexpr int kSmemBytes = kTileBytes + kVecBytes + 256 + 1024;
constexpr int kTmemCols = 512;                 // [S^T dP^T] x 2 | dK | dV
}  // namespace dkv

__global__ void __launch_bounds__(kThreads, 1)
flash_bwd_dkv_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                     const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                     const BwdParams p) {
  using namespace dkv;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t sK = base, sV = sK + kKBytes;
  const uint32_t sQ = sV + kKBytes;            // kQStages stages
  const uint32_t sDO = sQ + kQStages * kQBytes;
  const uint32_t sPT = sDO + kQStages * kQBytes, sDST = sPT + kPBytes;
  float* sLse = reinterpret_cast<float*>(gen + kTileBytes);       // [2][64]
  float* sDelta = sLse + 2 * kQT;                                  // [2][64]
  int* sLo = reinterpret_cast<int*>(sDelta + 2 * kQT);             // [2][64]
  int* sHi = sLo + 2 * kQT;                                        // [2][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + kTileBytes + kVecBytes);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_kv = bar0;
  const uint32_t bar_qfull = bar0 + 8, bar_qempty = bar0 + 40;      // up to 4 stages each
  const uint32_t bar_sfull = bar0 + 72, bar_sempty = bar0 + 88;
  const uint32_t bar_pfull = bar0 + 104, bar_pdone = bar0 + 112, bar_vec = bar0 + 120;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = blockIdx.y, b = blockIdx.z;
  const int k0 = blockIdx.x * kKeys;
  const int g = p.N / p.Kh;
  const int off = p.Lk - p.Lq;
  const int nqt = (p.Lq + kQT - 1) / kQT;
  int i_start = 0, i_end = nqt;
  if (p.causal) i_start = max(0, k0 - off) / kQT;
  const bool packed = p.seg_lo != nullptr;
  if (packed) {
    const long long rb = static_cast<long long>(b) * p.Lq;
    // queries past the segment of this tile's last key see none of its keys
    i_end = min(nqt, p.seg_hi[rb + min(k0 + kKeys, p.Lk) - 1] / kQT + 1);
    if (!p.causal) i_start = p.seg_lo[rb + k0] / kQT;
  }
  const int per_head = max(0, i_end - i_start);
  const int n_it = per_head * g;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_kv, 1);
    for (int s = 0; s < kQStages; ++s) {
      mbar_init(bar_qfull + 8 * s, 1);
      mbar_init(bar_qempty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_sfull + 8 * s, 1);
      mbar_init(bar_sempty + 8 * s, 256);
    }
    mbar_init(bar_pfull, 256);
    mbar_init(bar_pdone, 1);
    mbar_init(bar_vec, 256);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dk = tmem_base + 256, tmem_dv = tmem_base + 384;

  if (warp == 0) {
    if (elect_one() && n_it > 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_do);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const int krow = b * p.Lk + k0;
      mbar_expect_tx(bar_kv, 2 * kKBytes);
      tma_load_2d(sK, &map_k, kvh * kHD, krow, bar_kv);
      tma_load_2d(sK + kKeys * 128, &map_k, kvh * kHD + 64, krow, bar_kv);
      tma_load_2d(sV, &map_v, kvh * kHD, krow, bar_kv);
      tma_load_2d(sV + kKeys * 128, &map_v, kvh * kHD + 64, krow, bar_kv);
      for (int it = 0; it < n_it; ++it) {
        const int st = it % kQStages;
        const int h = kvh * g + it / per_head;
        const int qrow = b * p.Lq + (i_start + it % per_head) * kQT;
        if (!mbar_wait(bar_qempty + 8 * st, ((it / kQStages) & 1) ^ 1, abort_flag)) {
          atomicOr(p.status, kStatusWaitTimeoutProducer);
          break;
        }
        const uint32_t full = bar_qfull + 8 * st;
        mbar_expect_tx(full, 2 * kQBytes);
        tma_load_2d(sQ + st * kQBytes, &map_q, h * kHD, qrow, full);
        tma_load_2d(sQ + st * kQBytes + kQT * 128, &map_q, h * kHD + 64, qrow, full);
        tma_load_2d(sDO + st * kQBytes, &map_do, h * kHD, qrow, full);
        tma_load_2d(sDO + st * kQBytes + kQT * 128, &map_do, h * kHD + 64, qrow, full);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_it > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kKeys, kQT, false, false);
      constexpr uint32_t idesc_d = make_idesc_bf16(kKeys, kHD, false, true);
      bool ok = mbar_wait(bar_kv, 0, abort_flag);
      auto issue_sdp = [&](int it) -> bool {
        const int st = it & 1, qs = it % kQStages;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(bar_qfull + 8 * qs, (it / kQStages) & 1, abort_flag)) return false;
        if (!mbar_wait(bar_sempty + 8 * st, ph ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sq = sQ + qs * kQBytes, sdo = sDO + qs * kQBytes;
#pragma unroll
        for (int k = 0; k < kHD / 16; ++k) {
          const uint32_t sub = k >> 2, kk = k & 3;
          umma_bf16(tmem_base + st * 128, make_smem_desc_sw128(sK + sub * (kKeys * 128) + kk * 32, 16, 1024),
                    make_smem_desc_sw128(sq + sub * (kQT * 128) + kk * 32, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < kHD / 16; ++k) {
          const uint32_t sub = k >> 2, kk = k & 3;
          umma_bf16(tmem_base + st * 128 + 64, make_smem_desc_sw128(sV + sub * (kKeys * 128) + kk * 32, 16, 1024),
                    make_smem_desc_sw128(sdo + sub * (kQT * 128) + kk * 32, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(bar_sfull + 8 * st);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int it = 0; it < n_it && ok; ++it) {
        if (it + 1 < n_it) ok = issue_sdp(it + 1);
        if (!ok) break;
        const int st = it % kQStages;
        if (!mbar_wait(bar_pfull, it & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sq = sQ + st * kQBytes, sdo = sDO + st * kQBytes;
#pragma unroll
        for (int k = 0; k < kQT / 16; ++k)
          umma_bf16(tmem_dv, make_smem_desc_sw128(sPT + k * 32, 16, 1024),
                    make_smem_desc_sw128(sdo + k * 2048, kQT * 128, 1024), idesc_d, (it > 0 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < kQT / 16; ++k)
          umma_bf16(tmem_dk, make_smem_desc_sw128(sDST + k * 32, 16, 1024),
                    make_smem_desc_sw128(sq + k * 2048, kQT * 128, 1024), idesc_d, (it > 0 || k > 0) ? 1u : 0u);
        umma_commit(bar_qempty + 8 * st);
        umma_commit(bar_pdone);
      }
      if (!ok) atomicOr(p.status, kStatusWaitTimeoutMma);
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;           // key row in the tile == TMEM lane
    const int ch = (warp - 2) >> 2;              // which 32 of the 64 query columns this thread handles
    const int t256 = threadIdx.x - 64;           // 0..255 among the compute threads
    const int kj = k0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_it; ++it) {
      const int st = it & 1;
      const int h = kvh * g + it / per_head;
      const int q0 = (i_start + it % per_head) * kQT;
      {
        const int c = t256 & 63, which = t256 >> 6;
        const int qi = q0 + c;
        const long long idx = (static_cast<long long>(b) * p.N + h) * p.Lq + qi;
        if (which == 0) {
          float v = qi < p.Lq ? p.lse[idx] : INFINITY;
          sLse[st * kQT + c] = (v == -INFINITY) ? INFINITY : v * kLog2e;
        } else if (which == 1) {
          sLo[st * kQT + c] = (packed && qi < p.Lq) ? p.seg_lo[static_cast<long long>(b) * p.Lq + qi] : 0;
        } else if (which == 2) {
          sDelta[st * kQT + c] = qi < p.Lq ? p.delta[idx] : 0.f;
        } else {
          sHi[st * kQT + c] = (packed && qi < p.Lq) ? p.seg_hi[static_cast<long long>(b) * p.Lq + qi] : p.Lk - 1;
        }
      }
      // the 256 elementwise threads meet on a bounded barrier (a hardware bar.sync could not time out)
      mbar_arrive(bar_vec);
      ok = __all_sync(0xffffffffu, mbar_wait(bar_vec, it & 1, abort_flag));
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_sfull + 8 * st, (it >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      uint32_t pk[16], dk_[16];
      const bool need_mask = packed || (p.causal && k0 + kKeys - 1 > q0 + off) || (k0 + kKeys > p.Lk);
      {
        uint32_t ts[32], td[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + st * 128 + ch * 32, ts);
        tmem_ld_32x32b_x32(tmem_base + lane_addr + st * 128 + 64 + ch * 32, td);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pv[2], dv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int c = ch * 32 + i + e;
            float pe = exp2f(__uint_as_float(ts[i + e]) * p.scale_log2 - sLse[st * kQT + c]);
            if (need_mask && ((p.causal && kj > q0 + c + off) || kj >= p.Lk || kj < sLo[st * kQT + c] ||
                              kj > sHi[st * kQT + c]))
              pe = 0.f;
            pv[e] = pe;
            dv[e] = pe * (__uint_as_float(td[i + e]) - sDelta[st * kQT + c]);
          }
          pk[i >> 1] = pack2(pv[0], pv[1]);
          dk_[i >> 1] = pack2(dv[0], dv[1]);
        }
      }
      tc_fence_before();
      mbar_arrive(bar_sempty + 8 * st);
      if (it > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_pdone, (it - 1) & 1, abort_flag));
        if (!ok) break;
      }
      store_half_row_sw128(gen + (sPT - base), r, ch, pk);
      store_half_row_sw128(gen + (sDST - base), r, ch, dk_);
      fence_proxy_async_smem();
      mbar_arrive(bar_pfull);
    }
    if (ok && n_it > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar_pdone, (n_it - 1) & 1, abort_flag));
    if (!ok) atomicOr(p.status, kStatusWaitTimeoutEpilogue);
    if (ok) {
      tc_fence_after();
      const bool in_range = kj < p.Lk;
      const long long row = static_cast<long long>(b) * p.Lk + (in_range ? kj : 0);
      if (ch == 0) store_acc_rows(tmem_dk + lane_addr, p.out0 + row * p.ld0 + kvh * kHD, in_range, p.scale, n_it > 0);
      else         store_acc_rows(tmem_dv + lane_addr, p.out1 + row * p.ld1 + kvh * kHD, in_range, 1.f, n_it > 0);
    }
  }

  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------------------------------------------------
// dQ
// ------------------------------------------------------------------------------------------------
namespace dq {
constexpr int kBM = 128, kBN = 64;
constexpr int kQBytes = kBM * kHD * 2;         // 32 KiB
constexpr int kKVBytes = kBN * kHD * 2;        // 16 KiB
constexpr int kDSBytes = kBM * kBN * 2;        // 16 KiB
constexpr int kKVStages = 4;                   // K / V ring: a tile is requested three iterations ahead of its use
constexpr int kTileBytes = 2 * kQBytes + 2 * kKVStages * kKVBytes + kDSBytes;   // 212992
constexpr int kSmemBytes = kTileBytes + 256 + 1024;
constexpr int kTmemCols = 512;                 // [S dP] x 2 | dQ
}  // namespace dq

__global__ void __launch_bounds__(kThreads, 1)
flash_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const BwdParams p) {
  using namespace dq;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  const uint32_t sQ = base, sDO = sQ + kQBytes;
  const uint32_t sK = sDO + kQBytes;            // kKVStages stages
  const uint32_t sV = sK + kKVStages * kKVBytes;
  const uint32_t sDS = sV + kKVStages * kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + kTileBytes);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_q = bar0;
  const uint32_t bar_kvfull = bar0 + 8, bar_kvempty = bar0 + 40;    // up to 4 stages each
  const uint32_t bar_sfull = bar0 + 72, bar_sempty = bar0 + 88;
  const uint32_t bar_dsfull = bar0 + 104, bar_dsdone = bar0 + 112;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.Lq + kBM - 1) / kBM;
  const int qb = nqb - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.N / p.Kh);
  const int q0 = qb * kBM;
  const int off = p.Lk - p.Lq;
  int kv_end = p.Lk;
  if (p.causal) kv_end = min(p.Lk, q0 + kBM + off);
  int j0 = 0;
  if (p.seg_lo != nullptr) {
    const long long rb = static_cast<long long>(b) * p.Lq;
    j0 = p.seg_lo[rb + q0] / kBN;
    if (!p.causal) kv_end = min(p.Lk, p.seg_hi[rb + min(q0 + kBM, p.Lq) - 1] + 1);
  }
  const int n_tiles = kv_end > j0 * kBN ? (kv_end + kBN - 1) / kBN - j0 : 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q, 1);
    for (int s = 0; s < kKVStages; ++s) {
      mbar_init(bar_kvfull + 8 * s, 1);
      mbar_init(bar_kvempty + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_sfull + 8 * s, 1);
      mbar_init(bar_sempty + 8 * s, 256);
    }
    mbar_init(bar_dsfull, 256);
    mbar_init(bar_dsdone, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_dq = tmem_base + 256;

  if (warp == 0) {
    if (elect_one() && n_tiles > 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_do);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const int qrow = b * p.Lq + q0;
      mbar_expect_tx(bar_q, 2 * kQBytes);
      tma_load_2d(sQ, &map_q, h * kHD, qrow, bar_q);
      tma_load_2d(sQ + kBM * 128, &map_q, h * kHD + 64, qrow, bar_q);
      tma_load_2d(sDO, &map_do, h * kHD, qrow, bar_q);
      tma_load_2d(sDO + kBM * 128, &map_do, h * kHD + 64, qrow, bar_q);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % kKVStages;
        const int krow = b * p.Lk + (j0 + j) * kBN;
        if (!mbar_wait(bar_kvempty + 8 * st, ((j / kKVStages) & 1) ^ 1, abort_flag)) {
          atomicOr(p.status, kStatusWaitTimeoutProducer);
          break;
        }
        const uint32_t full = bar_kvfull + 8 * st;
        mbar_expect_tx(full, 2 * kKVBytes);
        tma_load_2d(sK + st * kKVBytes, &map_k, kvh * kHD, krow, full);
        tma_load_2d(sK + st * kKVBytes + kBN * 128, &map_k, kvh * kHD + 64, krow, full);
        tma_load_2d(sV + st * kKVBytes, &map_v, kvh * kHD, krow, full);
        tma_load_2d(sV + st * kKVBytes + kBN * 128, &map_v, kvh * kHD + 64, krow, full);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_tiles > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kBM, kBN, false, false);
      constexpr uint32_t idesc_d = make_idesc_bf16(kBM, kHD, false, true);
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      auto issue_sdp = [&](int j) -> bool {
        const int st = j & 1, ks = j % kKVStages;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(bar_kvfull + 8 * ks, (j / kKVStages) & 1, abort_flag)) return false;
        if (!mbar_wait(bar_sempty + 8 * st, ph ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sk = sK + ks * kKVBytes, sv = sV + ks * kKVBytes;
#pragma unroll
        for (int k = 0; k < kHD / 16; ++k) {
          const uint32_t sub = k >> 2, kk = k & 3;
          umma_bf16(tmem_base + st * 128, make_smem_desc_sw128(sQ + sub * (kBM * 128) + kk * 32, 16, 1024),
                    make_smem_desc_sw128(sk + sub * (kBN * 128) + kk * 32, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < kHD / 16; ++k) {
          const uint32_t sub = k >> 2, kk = k & 3;
          umma_bf16(tmem_base + st * 128 + 64, make_smem_desc_sw128(sDO + sub * (kBM * 128) + kk * 32, 16, 1024),
                    make_smem_desc_sw128(sv + sub * (kBN * 128) + kk * 32, 16, 1024), idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(bar_sfull + 8 * st);
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_sdp(j + 1);
        if (!ok) break;
        const int st = j % kKVStages;
        if (!mbar_wait(bar_dsfull, j & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sk = sK + st * kKVBytes;
#pragma unroll
        for (int k = 0; k < kBN / 16; ++k)
          umma_bf16(tmem_dq, make_smem_desc_sw128(sDS + k * 32, 16, 1024),
                    make_smem_desc_sw128(sk + k * 2048, kBN * 128, 1024), idesc_d, (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(bar_kvempty + 8 * st);
        umma_commit(bar_dsdone);
      }
      if (!ok) atomicOr(p.status, kStatusWaitTimeoutMma);
    }
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int ch = (warp - 2) >> 2;              // which 32 of the 64 key columns this thread handles
    const int qi = q0 + r;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float lse2 = INFINITY, delta = 0.f;
    if (qi < p.Lq) {
      const long long idx = (static_cast<long long>(b) * p.N + h) * p.Lq + qi;
      const float v = p.lse[idx];
      lse2 = (v == -INFINITY) ? INFINITY : v * kLog2e;
      delta = p.delta[idx];
    }
    int row_lo = 0, row_hi = p.Lk - 1;
    if (p.seg_lo != nullptr && qi < p.Lq) {
      row_lo = p.seg_lo[static_cast<long long>(b) * p.Lq + qi];
      row_hi = p.seg_hi[static_cast<long long>(b) * p.Lq + qi];
    }
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_sfull + 8 * st, (j >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const int k0 = (j0 + j) * kBN;
      const int limit = p.causal ? min(qi + off, row_hi) : row_hi;
      const bool need_mask = k0 + kBN - 1 > limit || k0 < row_lo;
      uint32_t dsk[16];
      {
        uint32_t ts[32], td[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + st * 128 + ch * 32, ts);
        tmem_ld_32x32b_x32(tmem_base + lane_addr + st * 128 + 64 + ch * 32, td);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float dv[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            float pe = exp2f(__uint_as_float(ts[i + e]) * p.scale_log2 - lse2);
            if (need_mask && (k0 + ch * 32 + i + e > limit || k0 + ch * 32 + i + e < row_lo)) pe = 0.f;
            dv[e] = pe * (__uint_as_float(td[i + e]) - delta);
          }
          dsk[i >> 1] = pack2(dv[0], dv[1]);
        }
      }
      tc_fence_before();
      mbar_arrive(bar_sempty + 8 * st);
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_dsdone, (j - 1) & 1, abort_flag));
        if (!ok) break;
      }
      store_half_row_sw128(gen + (sDS - base), r, ch, dsk);
      fence_proxy_async_smem();
      mbar_arrive(bar_dsfull);
    }
    if (ok && n_tiles > 0) ok = __all_sync(0xffffffffu, mbar_wait(bar_dsdone, (n_tiles - 1) & 1, abort_flag));
    if (!ok) atomicOr(p.status, kStatusWaitTimeoutEpilogue);
    if (ok) {
      tc_fence_after();
      const bool in_range = qi < p.Lq;
      const long long row = static_cast<long long>(b) * p.Lq + (in_range ? qi : 0);
      store_acc_rows(tmem_dq + lane_addr, p.out0 + row * p.ld0 + h * kHD, in_range, p.scale, n_tiles > 0, ch * 64,
                     ch * 64 + 64);
    }
  }

  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace

// dq/dk/dv/q/k/v/o/d_o: bf16, row strides in elements (multiples of 8). `delta` is caller-provided
// scratch of B*N*Lq floats. Returns 0, 1 for an unsupported shape, 3xx tensor-map failure, 400 launch.
extern "C" int tx_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, void* dq_out, void* dk_out, void* dv_out, int B, int N,
                            int Kh, int Lq, int Lk, int head_dim, long long ldq, long long ldk, long long ldv,
                            long long ldo, long long lddo, long long lddq, long long lddk, long long lddv,
                            int causal, float scale, int* status, cudaStream_t stream);

// As tx_flash_bwd for packed rows (seg_lo / seg_hi int32 [B, Lq], both or neither; need Lq == Lk).
extern "C" int tx_flash_bwd_seg(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                const float* lse, float* delta, void* dq_out, void* dk_out, void* dv_out, int B,
                                int N, int Kh, int Lq, int Lk, int head_dim, long long ldq, long long ldk,
                                long long ldv, long long ldo, long long lddo, long long lddq, long long lddk,
                                long long lddv, int causal, float scale, const int* seg_lo, const int* seg_hi,
                                int* status, cudaStream_t stream) {
  if ((seg_lo == nullptr) != (seg_hi == nullptr) || (seg_lo != nullptr && Lq != Lk)) return 1;
  if (head_dim != kHD || B <= 0 || N <= 0 || Kh <= 0 || N % Kh != 0 || Lq <= 0 || Lk <= 0) return 1;
  if ((ldq | ldk | ldv | ldo | lddo | lddq | lddk | lddv) % 8 != 0) return 1;
  const uint64_t rq = static_cast<uint64_t>(B) * Lq, rk = static_cast<uint64_t>(B) * Lk;
  const uint64_t cq = static_cast<uint64_t>(N) * kHD, ck = static_cast<uint64_t>(Kh) * kHD;
  CUtensorMap q64, do64, k128, v128, q128, do128, k64, v64;
  int rc = txh::make_map_2d_bf16(&q64, q, rq, cq, ldq, 64, 64);
  if (!rc) rc = txh::make_map_2d_bf16(&do64, d_o, rq, cq, lddo, 64, 64);
  if (!rc) rc = txh::make_map_2d_bf16(&k128, k, rk, ck, ldk, 128, 64);
  if (!rc) rc = txh::make_map_2d_bf16(&v128, v, rk, ck, ldv, 128, 64);
  if (!rc) rc = txh::make_map_2d_bf16(&q128, q, rq, cq, ldq, 128, 64);
  if (!rc) rc = txh::make_map_2d_bf16(&do128, d_o, rq, cq, lddo, 128, 64);
  if (!rc) rc = txh::make_map_2d_bf16(&k64, k, rk, ck, ldk, 64, 64);
  if (!rc) rc = txh::make_map_2d_bf16(&v64, v, rk, ck, ldv, 64, 64);
  if (rc) return 300 + rc;
  static txh::DeviceFlag attr_flag;
  bool& attr_set = attr_flag.cur();
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dkv::kSmemBytes) !=
            cudaSuccess ||
        cudaFuncSetAttribute(flash_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, dq::kSmemBytes) !=
            cudaSuccess)
      return 400;
    attr_set = true;
  }
  const long long warps = static_cast<long long>(B) * Lq * N;
  flash_bwd_delta_kernel<<<static_cast<unsigned>((warps + 7) / 8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, ldo, lddo, B, N, Lq);
  BwdParams p;
  p.lse = lse;
  p.delta = delta;
  p.B = B; p.N = N; p.Kh = Kh; p.Lq = Lq; p.Lk = Lk; p.causal = causal;
  p.scale = scale;
  p.scale_log2 = scale * kLog2e;
  p.status = status;
  p.seg_lo = seg_lo;
  p.seg_hi = seg_hi;
  p.out0 = static_cast<__nv_bfloat16*>(dk_out);
  p.out1 = static_cast<__nv_bfloat16*>(dv_out);
  p.ld0 = lddk;
  p.ld1 = lddv;
  dim3 gkv((Lk + dkv::kKeys - 1) / dkv::kKeys, Kh, B);
  flash_bwd_dkv_kernel<<<gkv, kThreads, dkv::kSmemBytes, stream>>>(q64, do64, k128, v128, p);
  p.out0 = static_cast<__nv_bfloat16*>(dq_out);
  p.out1 = nullptr;
  p.ld0 = lddq;
  p.ld1 = 0;
  dim3 gq((Lq + dq::kBM - 1) / dq::kBM, N, B);
  flash_bwd_dq_kernel<<<gq, kThreads, dq::kSmemBytes, stream>>>(q128, do128, k64, v64, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

extern "C" int tx_flash_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                            const float* lse, float* delta, void* dq_out, void* dk_out, void* dv_out, int B, int N,
                            int Kh, int Lq, int Lk, int head_dim, long long ldq, long long ldk, long long ldv,
                            long long ldo, long long lddo, long long lddq, long long lddk, long long lddv,
                            int causal, float scale, int* status, cudaStream_t stream) {
  return tx_flash_bwd_seg(q, k, v, o, d_o, lse, delta, dq_out, dk_out, dv_out, B, N, Kh, Lq, Lk, head_dim, ldq, ldk,
                          ldv, ldo, lddo, lddq, lddk, lddv, causal, scale, nullptr, nullptr, status, stream);
}
