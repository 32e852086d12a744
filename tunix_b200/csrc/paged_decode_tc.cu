// Paged decode attention on tcgen05 tensor cores (head_dim 128, GQA groups of up to 32 heads).
//
// One CTA per (split, kv head, sequence). The G = N / Kh query heads that share a kv head are
// the first G rows of a 128-row MMA tile; the other rows are zero and ignored. The tensor cores
// are nearly idle either way (decode is bound by reading K and V once), so the padded rows cost
// nothing, while the per-key work of the CUDA cores drops from ~80 warp instructions (dot
// products, shuffles and online-softmax updates in the SIMT kernel) to ~6.
//
//   warp 0  softmax: lane g owns query head g (TMEM lane g): reads S, running max / sum,
//           writes P (bf16, 128-byte swizzled) to shared memory, lazily rescales O in TMEM,
//           normalises and stores at the end (or writes the split's partial to the workspace)
//   warp 1  MMA issuer: S = Q K^T into one of two TMEM buffers, O += P V
//   warp 2  TMA producer: one box per page (page_size rows x 64 dims) through 2-stage K and V
//           rings; pages come from the sequence's block table; boxes past the sequence's last
//           page are fetched from an out-of-range row so they arrive as zeros
//   warp 3  helps stage Q
//
// 112 KiB of shared memory and 256 TMEM columns per CTA: two CTAs per SM. Every wait is
// bounded; a timeout sets a status bit and all roles leave their loops.
//
// The cache pages must hold finite values everywhere (they are zero-initialised and only ever
// written with projections): a masked key contributes 0 * v, which must not be NaN.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "tx_host.h"
#include "tx_ptx.cuh"

namespace {
using namespace tx;

constexpr int kHD = 128;
constexpr int kBM = 128;
constexpr int kBN = 64;
constexpr int kThreads = 128;
constexpr int kQBytes = kBM * kHD * 2;
constexpr int kKVBytes = kBN * kHD * 2;
constexpr int kPBytes = kBM * kBN * 2;
constexpr int kStages = 2;
constexpr int kTileBytes = kQBytes + 2 * kStages * kKVBytes + kPBytes;   // 114688
constexpr int kBarBytes = 256;
constexpr int kSmemBytes = kTileBytes + kBarBytes + 768;
constexpr int kTmemCols = 256;                  // S0 [0,64) S1 [64,128) O [128,256)
constexpr float kRescaleThreshold = 8.f;

struct DecodeParams {
  const __nv_bfloat16* q;
  long long ldq;
  const int* block_tables;
  int max_blocks;
  const int* seq_lens;
  int page_size;
  int total_rows;     // pages * page_size: the first out-of-range row of the K/V maps
  int Kh, G;
  float scale_log2;
  int num_splits;
  float* ws_o;
  float* ws_ml;
  __nv_bfloat16* out;
  long long ldo;
  int* status;
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__global__ void __launch_bounds__(kThreads, 2)
paged_decode_tc_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const DecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  if (base - raw + kTileBytes + kBarBytes > kSmemBytes) {
    if (threadIdx.x == 0) atomicOr(p.status, kStatusBadArgument);
    return;
  }
  const uint32_t sQ = base;
  const uint32_t sK = sQ + kQBytes;
  const uint32_t sV = sK + kStages * kKVBytes;
  const uint32_t sP = sV + kStages * kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + kTileBytes);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_kfull = bar0 + 8, bar_kempty = bar0 + 24;
  const uint32_t bar_vfull = bar0 + 40, bar_vempty = bar0 + 56;
  const uint32_t bar_sfull = bar0 + 72, bar_sempty = bar0 + 88;
  const uint32_t bar_pfull = bar0 + 104, bar_pvdone = bar0 + 112;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int G = p.G, N = p.Kh * G;
  const int len = p.seq_lens[b];
  // this split's keys: whole tiles of 64, [lo, hi)
  const int tiles_total = (len + kBN - 1) / kBN;
  const int tiles_per = (tiles_total + p.num_splits - 1) / p.num_splits;
  const int lo = min(len, split * tiles_per * kBN);
  const int hi = min(len, lo + tiles_per * kBN);
  const int n_tiles = (hi - lo + kBN - 1) / kBN;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_kempty + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_vempty + 8 * s, 1);
      mbar_init(bar_sfull + 8 * s, 1);
      mbar_init(bar_sempty + 8 * s, 32);
    }
    mbar_init(bar_pfull, 32);
    mbar_init(bar_pvdone, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  // Stage Q: zero the tile, then rows 0..G-1 (two swizzled [128 x 64] sub-tiles).
  {
    uint4* qz = reinterpret_cast<uint4*>(gen);
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    for (int i = threadIdx.x; i < kQBytes / 16; i += kThreads) qz[i] = z;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * 16; i += kThreads) {
    const int g = i >> 4, c16 = i & 15, sub = c16 >> 3, c = c16 & 7;
    const uint4 v4 = *reinterpret_cast<const uint4*>(p.q + static_cast<long long>(b) * p.ldq +
                                                     static_cast<long long>(kvh * G + g) * kHD + c16 * 8);
    *reinterpret_cast<uint4*>(gen + sub * (kBM * 128) + g * 128 + ((c ^ (g & 7)) << 4)) = v4;
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128;

  if (warp == 2) {
    if (elect_one() && n_tiles > 0) {
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const int page = p.page_size;
      const int boxes = kBN / page;                         // pages per tile (page divides 64)
      const int n_pages = (len + page - 1) / page;          // pages this sequence owns
      const int* bt = p.block_tables + static_cast<long long>(b) * p.max_blocks;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int page0 = (lo + j * kBN) / page;
        if (!mbar_wait(bar_kempty + 8 * st, ph ^ 1, abort_flag)) {
          atomicOr(p.status, kStatusWaitTimeoutProducer);
          break;
        }
        mbar_expect_tx(bar_kfull + 8 * st, kKVBytes);
        for (int i = 0; i < boxes; ++i) {
          const int pg = page0 + i;
          const int row = (pg < n_pages && pg < p.max_blocks) ? bt[pg] * page : p.total_rows;
          const uint32_t dst = sK + st * kKVBytes + i * page * 128;
          tma_load_2d(dst, &map_k, kvh * kHD, row, bar_kfull + 8 * st);
          tma_load_2d(dst + kBN * 128, &map_k, kvh * kHD + 64, row, bar_kfull + 8 * st);
        }
        if (!mbar_wait(bar_vempty + 8 * st, ph ^ 1, abort_flag)) {
          atomicOr(p.status, kStatusWaitTimeoutProducer);
          break;
        }
        mbar_expect_tx(bar_vfull + 8 * st, kKVBytes);
        for (int i = 0; i < boxes; ++i) {
          const int pg = page0 + i;
          const int row = (pg < n_pages && pg < p.max_blocks) ? bt[pg] * page : p.total_rows;
          const uint32_t dst = sV + st * kKVBytes + i * page * 128;
          tma_load_2d(dst, &map_v, kvh * kHD, row, bar_vfull + 8 * st);
          tma_load_2d(dst + kBN * 128, &map_v, kvh * kHD + 64, row, bar_vfull + 8 * st);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_tiles > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kBM, kBN, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(kBM, kHD, false, true);
      bool ok = true;
      auto issue_qk = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(bar_kfull + 8 * st, ph, abort_flag)) return false;
        if (!mbar_wait(bar_sempty + 8 * st, ph ^ 1, abort_flag)) return false;
        tc_fence_after();
        const uint32_t sk = sK + st * kKVBytes;
#pragma unroll
        for (int k = 0; k < kHD / 16; ++k) {
          const uint32_t sub = (k >> 2), kk = (k & 3);
          const uint64_t da = make_smem_desc_sw128(sQ + sub * (kBM * 128) + kk * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sk + sub * (kBN * 128) + kk * 32, 16, 1024);
          umma_bf16(tmem_base + st * kBN, da, db, idesc_s, k > 0 ? 1u : 0u);
        }
        umma_commit(bar_kempty + 8 * st);
        umma_commit(bar_sfull + 8 * st);
        return true;
      };
      ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);
        if (!ok) break;
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(bar_vfull + 8 * st, ph, abort_flag) || !mbar_wait(bar_pfull, j & 1, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t sv = sV + st * kKVBytes;
#pragma unroll
        for (int k = 0; k < kBN / 16; ++k) {
          const uint64_t da = make_smem_desc_sw128(sP + k * 32, 16, 1024);
          const uint64_t db = make_smem_desc_sw128(sv + k * 2048, kBN * 128, 1024);
          umma_bf16(tmem_o, da, db, idesc_o, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(bar_vempty + 8 * st);
        umma_commit(bar_pvdone);
      }
      if (!ok) atomicOr(p.status, kStatusWaitTimeoutMma);
    }
  } else if (warp == 0) {
    const int r = lane;                            // row of the tile == TMEM lane == query head in the group
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    // rows G..31 of P stay zero: clear the first 32 rows once
    {
      uint4* pz = reinterpret_cast<uint4*>(gen + (sP - base));
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      for (int i = lane; i < 32 * 128 / 16; i += 32) pz[i] = z;
      __syncwarp();
    }
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_sfull + 8 * st, (j >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      float s[kBN];
      {
        uint32_t t0[32], t1[32];
        tmem_ld_32x32b_x32(tmem_base + st * kBN, t0);
        tmem_ld_32x32b_x32(tmem_base + st * kBN + 32, t1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          s[i] = __uint_as_float(t0[i]) * p.scale_log2;
          s[32 + i] = __uint_as_float(t1[i]) * p.scale_log2;
        }
      }
      tc_fence_before();
      mbar_arrive(bar_sempty + 8 * st);
      const int k0 = lo + j * kBN;
      if (k0 + kBN > hi) {
#pragma unroll
        for (int i = 0; i < kBN; ++i)
          if (k0 + i >= hi) s[i] = -INFINITY;
      }
      float mt = s[0];
#pragma unroll
      for (int i = 1; i < kBN; ++i) mt = fmaxf(mt, s[i]);
      float alpha = 1.f;
      bool need = false;
      if (mt > m_ref + kRescaleThreshold) {
        alpha = exp2f(m_ref - mt);
        m_ref = mt;
        need = j > 0 && r < G;
      }
      const float mu = (m_ref == -INFINITY) ? 0.f : m_ref;
      float rs = 0.f;
      uint32_t pk[kBN / 2];
#pragma unroll
      for (int i = 0; i < kBN; i += 2) {
        const float e0 = exp2f(s[i] - mu), e1 = exp2f(s[i + 1] - mu);
        rs += e0 + e1;
        pk[i >> 1] = pack_bf16(e0, e1);
      }
      l = l * alpha + rs;
      if (j > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_pvdone, (j - 1) & 1, abort_flag));
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, need)) {
#pragma unroll 1
          for (int c = 0; c < kHD; c += 16) {
            uint32_t t[16];
            tmem_ld_32x32b_x16(tmem_o + c, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
            tmem_st_32x32b_x16(tmem_o + c, t);
          }
          tmem_st_wait();
        }
      }
      if (r < G) {
        uint8_t* prow = gen + (sP - base) + r * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 v4 = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
          *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = v4;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(bar_pfull);
    }
    if (ok && n_tiles > 0)
      ok = __all_sync(0xffffffffu, mbar_wait(bar_pvdone, (n_tiles - 1) & 1, abort_flag));
    if (!ok) atomicOr(p.status, kStatusWaitTimeoutEpilogue);
    if (ok) {
      tc_fence_after();
      const bool valid = r < G;
      const int head = kvh * G + (valid ? r : 0);
      const long long wbase = (static_cast<long long>(b) * N + head) * p.num_splits + split;
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
      for (int c = 0; c < kHD; c += 32) {
        uint32_t t[32];
        if (n_tiles > 0) {
          tmem_ld_32x32b_x32(tmem_o + c, t);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = 0u;
        }
        if (valid) {
          if (p.num_splits == 1) {
            __nv_bfloat16* orow = p.out + static_cast<long long>(b) * p.ldo + static_cast<long long>(head) * kHD;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v4;
              v4.x = pack_bf16(__uint_as_float(t[i]) * inv, __uint_as_float(t[i + 1]) * inv);
              v4.y = pack_bf16(__uint_as_float(t[i + 2]) * inv, __uint_as_float(t[i + 3]) * inv);
              v4.z = pack_bf16(__uint_as_float(t[i + 4]) * inv, __uint_as_float(t[i + 5]) * inv);
              v4.w = pack_bf16(__uint_as_float(t[i + 6]) * inv, __uint_as_float(t[i + 7]) * inv);
              *reinterpret_cast<uint4*>(orow + c + i) = v4;
            }
          } else {
            float4* wo = reinterpret_cast<float4*>(p.ws_o + wbase * kHD + c);
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              wo[i >> 2] = make_float4(__uint_as_float(t[i]), __uint_as_float(t[i + 1]), __uint_as_float(t[i + 2]),
                                       __uint_as_float(t[i + 3]));
          }
        }
      }
      if (valid && p.num_splits > 1) {
        p.ws_ml[wbase * 2] = m_ref;
        p.ws_ml[wbase * 2 + 1] = l;
      }
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

// Tensor-core paged decode attention. Shapes as tx_paged_decode_attn; restrictions: H == 128,
// page_size in {8, 16, 32, 64}, G = N / Kh <= 32, ldq and ldo multiples of 8. With num_splits > 1 the
// partial results go to ws_o [B*N*splits*128] / ws_ml [B*N*splits*2] in the layout the combine kernel
// of tx_paged_decode_attn reads; the caller runs tx_paged_decode_combine afterwards.
// Returns 0, 1 for an unsupported shape, 3xx for a tensor-map failure, 400 for a refused launch.
extern "C" int tx_paged_decode_attn_tc(const void* q, long long ldq, const void* k_pages, const void* v_pages,
                                       const int* block_tables, int max_blocks, const int* seq_lens, int B, int N,
                                       int Kh, int H, int page_size, long long num_pages, float scale,
                                       int num_splits, float* ws_o, float* ws_ml, void* out, long long ldo,
                                       int* status, cudaStream_t stream) {
  if (H != kHD || B <= 0 || Kh <= 0 || N % Kh != 0 || N / Kh > 32 || num_splits < 1) return 1;
  if (page_size != 8 && page_size != 16 && page_size != 32 && page_size != 64) return 1;
  if ((ldq | ldo) % 8 != 0 || (num_splits > 1 && (!ws_o || !ws_ml))) return 1;
  if (num_pages <= 0 || num_pages * page_size > 0x7fffffffLL) return 1;
  CUtensorMap mk, mv;
  const uint64_t rows = static_cast<uint64_t>(num_pages) * page_size;
  const uint64_t cols = static_cast<uint64_t>(Kh) * kHD;
  int rc = txh::make_map_2d_bf16(&mk, k_pages, rows, cols, cols, page_size, 64);
  if (rc == 0) rc = txh::make_map_2d_bf16(&mv, v_pages, rows, cols, cols, page_size, 64);
  if (rc != 0) return 300 + rc;
  static txh::DeviceFlag attr_flag;
  bool& attr_set = attr_flag.cur();
  if (!attr_set) {
    if (cudaFuncSetAttribute(paged_decode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
        cudaSuccess)
      return 400;
    attr_set = true;
  }
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.ldq = ldq;
  p.block_tables = block_tables;
  p.max_blocks = max_blocks;
  p.seq_lens = seq_lens;
  p.page_size = page_size;
  p.total_rows = static_cast<int>(rows);
  p.Kh = Kh;
  p.G = N / Kh;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_splits = num_splits;
  p.ws_o = ws_o;
  p.ws_ml = ws_ml;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ldo = ldo;
  p.status = status;
  dim3 grid(num_splits, Kh, B);
  paged_decode_tc_kernel<<<grid, kThreads, kSmemBytes, stream>>>(mk, mv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}
