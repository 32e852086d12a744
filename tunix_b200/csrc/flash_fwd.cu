// Causal / full flash attention forward for head_dim 128 on tcgen05 tensor cores.
//
// One CTA per (128 query rows, head, batch). Roles, as in the GEMM of this library:
//   warp 0      TMA producer: Q once, then K and V tiles of 64 keys through 2-stage rings
//   warp 1      MMA issuer:   S = Q K^T into one of two TMEM buffers, O += P V into TMEM
//   warps 2..5  softmax: one thread per query row (TMEM lane); reads S, keeps the running
//               max / sum, writes P (bf16, 128-byte swizzled) to shared memory, rescales O in
//               TMEM only when the running max moved by more than 2^8, normalises and stores
//               O and the log-sum-exp at the end.
// The CTA needs 112 KiB of shared memory and 256 TMEM columns, so two CTAs share an SM and one
// CTA's softmax overlaps the other's MMAs. All waits are bounded; a timeout sets a bit in the
// status word and every role leaves its loop.
//
// Layout: q [B*Lq, ldq] with head h at columns [h*128, h*128+128); k, v [B*Lk, ld] likewise
// (q, k and v may be views of one fused projection output); o [B*Lq, ldo]; lse [B, N, Lq] fp32
// (natural log). Causal masking is bottom-right aligned (key j visible to query i when
// j <= i + Lk - Lq).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "tx_host.h"
#include "tx_ptx.cuh"

namespace {
using namespace tx;

constexpr int kHD = 128;      // head dim
constexpr int kBM = 128;      // query rows per CTA
constexpr int kBN = 64;       // keys per tile
constexpr int kThreads = 192;
constexpr int kQBytes = kBM * kHD * 2;          // 32 KiB: two [128 x 64] swizzled sub-tiles
constexpr int kKVBytes = kBN * kHD * 2;         // 16 KiB: two [64 x 64] sub-tiles
constexpr int kPBytes = kBM * kBN * 2;          // 16 KiB
constexpr int kStages = 2;
constexpr int kTileBytes = kQBytes + 2 * kStages * kKVBytes + kPBytes;   // 114688
constexpr int kBarBytes = 256;
constexpr int kSmemBytes = kTileBytes + kBarBytes + 768;                  // 115712: two CTAs per SM
constexpr int kTmemCols = 256;                  // S0 [0,64) S1 [64,128) O [128,256)
constexpr float kRescaleThreshold = 8.f;        // log2 units

struct FlashParams {
  __nv_bfloat16* o;
  float* lse;
  long long ldo;
  int B, N, Kh, Lq, Lk;
  int causal;
  float scale_log2;   // softmax scale * log2(e)
  int* status;
  // Packed sequences (optional, need Lq == Lk): per token the first and last index of its segment.
  // Key k is visible to query q when seg_lo[q] <= k <= (causal ? q : seg_hi[q]).
  const int* seg_lo;
  const int* seg_hi;
};

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__global__ void __launch_bounds__(kThreads, 2)
flash_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const FlashParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - raw);
  if (base - raw + kTileBytes + kBarBytes > kSmemBytes) {   // cannot happen with a 256-byte aligned base
    if (threadIdx.x == 0) atomicOr(p.status, kStatusBadArgument);
    return;
  }
  const uint32_t sQ = base;
  const uint32_t sK = sQ + kQBytes;
  const uint32_t sV = sK + kStages * kKVBytes;
  const uint32_t sP = sV + kStages * kKVBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(gen + kTileBytes);
  const uint32_t bar0 = smem_u32(bars);
  const uint32_t bar_q = bar0;
  const uint32_t bar_kfull = bar0 + 8, bar_kempty = bar0 + 24;
  const uint32_t bar_vfull = bar0 + 40, bar_vempty = bar0 + 56;
  const uint32_t bar_sfull = bar0 + 72, bar_sempty = bar0 + 88;
  const uint32_t bar_pfull = bar0 + 104, bar_pvdone = bar0 + 112;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = (p.Lq + kBM - 1) / kBM;
  const int qb = nqb - 1 - blockIdx.x;         // long rows first
  const int h = blockIdx.y, b = blockIdx.z;
  const int kvh = h / (p.N / p.Kh);
  const int q0 = qb * kBM;
  const int off = p.Lk - p.Lq;
  int kv_end = p.Lk;
  if (p.causal) kv_end = min(p.Lk, q0 + kBM + off);
  int j0 = 0;                                   // first key tile any row of this CTA can see
  if (p.seg_lo != nullptr) {
    const long long rb = static_cast<long long>(b) * p.Lq;
    j0 = p.seg_lo[rb + q0] / kBN;               // seg_lo is non-decreasing along the sequence
    if (!p.causal) kv_end = min(p.Lk, p.seg_hi[rb + min(q0 + kBM, p.Lq) - 1] + 1);
  }
  const int n_tiles = kv_end > j0 * kBN ? (kv_end + kBN - 1) / kBN - j0 : 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_kfull + 8 * s, 1);
      mbar_init(bar_kempty + 8 * s, 1);
      mbar_init(bar_vfull + 8 * s, 1);
      mbar_init(bar_vempty + 8 * s, 1);
      mbar_init(bar_sfull + 8 * s, 1);
      mbar_init(bar_sempty + 8 * s, 128);
    }
    mbar_init(bar_pfull, 128);
    mbar_init(bar_pvdone, 1);
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
  const uint32_t tmem_o = tmem_base + 128;

  if (warp == 0) {
    if (elect_one() && n_tiles > 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const int qrow = b * p.Lq + q0;
      mbar_expect_tx(bar_q, kQBytes);
      tma_load_2d(sQ, &map_q, h * kHD, qrow, bar_q);
      tma_load_2d(sQ + kBM * 128, &map_q, h * kHD + 64, qrow, bar_q);
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int krow = b * p.Lk + (j0 + j) * kBN;
        if (!mbar_wait(bar_kempty + 8 * st, ph ^ 1, abort_flag)) {
          atomicOr(p.status, kStatusWaitTimeoutProducer);
          break;
        }
        mbar_expect_tx(bar_kfull + 8 * st, kKVBytes);
        tma_load_2d(sK + st * kKVBytes, &map_k, kvh * kHD, krow, bar_kfull + 8 * st);
        tma_load_2d(sK + st * kKVBytes + kBN * 128, &map_k, kvh * kHD + 64, krow, bar_kfull + 8 * st);
        if (!mbar_wait(bar_vempty + 8 * st, ph ^ 1, abort_flag)) {
          atomicOr(p.status, kStatusWaitTimeoutProducer);
          break;
        }
        mbar_expect_tx(bar_vfull + 8 * st, kKVBytes);
        tma_load_2d(sV + st * kKVBytes, &map_v, kvh * kHD, krow, bar_vfull + 8 * st);
        tma_load_2d(sV + st * kKVBytes + kBN * 128, &map_v, kvh * kHD + 64, krow, bar_vfull + 8 * st);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && n_tiles > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(kBM, kBN, false, false);
      constexpr uint32_t idesc_o = make_idesc_bf16(kBM, kHD, false, true);
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      // S(j) = Q K_j^T into S buffer j&1
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
      if (ok) ok = issue_qk(0);
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
  } else {
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;            // row within the tile == TMEM lane
    const int qi = q0 + r;                        // query index within the sequence
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    int row_lo = 0, row_hi = p.Lk - 1;            // this row's segment (whole sequence without packing)
    if (p.seg_lo != nullptr && qi < p.Lq) {
      row_lo = p.seg_lo[static_cast<long long>(b) * p.Lq + qi];
      row_hi = p.seg_hi[static_cast<long long>(b) * p.Lq + qi];
    }
    for (int j = 0; j < n_tiles; ++j) {
      const int st = j & 1;
      // every decision that guards a warp-collective TMEM access is made warp-uniform
      ok = __all_sync(0xffffffffu, mbar_wait(bar_sfull + 8 * st, (j >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      float s[kBN];
      {
        uint32_t t0[32], t1[32];
        tmem_ld_32x32b_x32(tmem_base + lane_addr + st * kBN, t0);
        tmem_ld_32x32b_x32(tmem_base + lane_addr + st * kBN + 32, t1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          s[i] = __uint_as_float(t0[i]) * p.scale_log2;
          s[32 + i] = __uint_as_float(t1[i]) * p.scale_log2;
        }
      }
      tc_fence_before();
      mbar_arrive(bar_sempty + 8 * st);
      const int k0 = (j0 + j) * kBN;
      const int limit = p.causal ? min(qi + off, row_hi) : row_hi;       // last visible key
      if (k0 + kBN - 1 > limit) {
#pragma unroll
        for (int i = 0; i < kBN; ++i)
          if (k0 + i > limit) s[i] = -INFINITY;
      }
      if (k0 < row_lo) {                                                 // keys of earlier segments
#pragma unroll
        for (int i = 0; i < kBN; ++i)
          if (k0 + i < row_lo) s[i] = -INFINITY;
      }
      float mt = s[0];
#pragma unroll
      for (int i = 1; i < kBN; ++i) mt = fmaxf(mt, s[i]);
      float alpha = 1.f;
      bool need = false;
      if (mt > m_ref + kRescaleThreshold) {        // also true on the first tile (m_ref = -inf)
        alpha = exp2f(m_ref - mt);                  // 0 on the first tile
        m_ref = mt;
        need = j > 0;
      }
      const float mu = (m_ref == -INFINITY) ? 0.f : m_ref;   // fully masked row: keep exp2 finite
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
            tmem_ld_32x32b_x16(tmem_o + lane_addr + c, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
            tmem_st_32x32b_x16(tmem_o + lane_addr + c, t);
          }
          tmem_st_wait();
        }
      }
      // P row r: eight 16-byte chunks, chunk c stored at position c ^ (r & 7) of its 128-byte row
      uint8_t* prow = gen + (sP - base) + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 v4 = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        *reinterpret_cast<uint4*>(prow + ((c ^ (r & 7)) << 4)) = v4;
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
      const bool in_range = qi < p.Lq;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.o + (static_cast<long long>(b) * p.Lq + (in_range ? qi : 0)) * p.ldo + h * kHD;
#pragma unroll 1
      for (int c = 0; c < kHD; c += 32) {
        uint32_t t[32];
        if (n_tiles > 0) {                       // uniform over the CTA
          tmem_ld_32x32b_x32(tmem_o + lane_addr + c, t);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = 0u;
        }
        if (in_range) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 v4;
            v4.x = pack_bf16(__uint_as_float(t[i]) * inv, __uint_as_float(t[i + 1]) * inv);
            v4.y = pack_bf16(__uint_as_float(t[i + 2]) * inv, __uint_as_float(t[i + 3]) * inv);
            v4.z = pack_bf16(__uint_as_float(t[i + 4]) * inv, __uint_as_float(t[i + 5]) * inv);
            v4.w = pack_bf16(__uint_as_float(t[i + 6]) * inv, __uint_as_float(t[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c + i) = v4;
          }
        }
      }
      if (in_range)
        p.lse[(static_cast<long long>(b) * p.N + h) * p.Lq + qi] =
            l > 0.f ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
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

// q/k/v/o: bf16 device pointers, row strides in elements (multiples of 8, 16-byte aligned bases).
// Returns 0, 1 for an unsupported shape, 3xx for a tensor-map failure, 400 for a refused launch.
extern "C" int tx_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int N,
                            int Kh, int Lq, int Lk, int head_dim, long long ldq, long long ldk, long long ldv,
                            long long ldo, int causal, float scale, int* status, cudaStream_t stream);

// As tx_flash_fwd, for packed rows: seg_lo / seg_hi are int32 [B, Lq] (first / last token index of each
// token's segment, both nullptr for unpacked rows); they need Lq == Lk.
extern "C" int tx_flash_fwd_seg(const void* q, const void* k, const void* v, void* o, float* lse, int B, int N,
                                int Kh, int Lq, int Lk, int head_dim, long long ldq, long long ldk, long long ldv,
                                long long ldo, int causal, float scale, const int* seg_lo, const int* seg_hi,
                                int* status, cudaStream_t stream) {
  if ((seg_lo == nullptr) != (seg_hi == nullptr) || (seg_lo != nullptr && Lq != Lk)) return 1;
  if (head_dim != kHD || B <= 0 || N <= 0 || Kh <= 0 || N % Kh != 0 || Lq <= 0 || Lk <= 0) return 1;
  if ((ldq | ldk | ldv | ldo) % 8 != 0) return 1;
  CUtensorMap mq, mk, mv;
  int rc = txh::make_map_2d_bf16(&mq, q, static_cast<uint64_t>(B) * Lq, static_cast<uint64_t>(N) * kHD, ldq, kBM, 64);
  if (rc == 0) rc = txh::make_map_2d_bf16(&mk, k, static_cast<uint64_t>(B) * Lk, static_cast<uint64_t>(Kh) * kHD, ldk, kBN, 64);
  if (rc == 0) rc = txh::make_map_2d_bf16(&mv, v, static_cast<uint64_t>(B) * Lk, static_cast<uint64_t>(Kh) * kHD, ldv, kBN, 64);
  if (rc != 0) return 300 + rc;
  static txh::DeviceFlag attr_flag;
  bool& attr_set = attr_flag.cur();
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) !=
        cudaSuccess)
      return 400;
    attr_set = true;
  }
  FlashParams p;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.ldo = ldo;
  p.B = B; p.N = N; p.Kh = Kh; p.Lq = Lq; p.Lk = Lk;
  p.causal = causal;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = status;
  p.seg_lo = seg_lo;
  p.seg_hi = seg_hi;
  dim3 grid((Lq + kBM - 1) / kBM, N, B);
  flash_fwd_kernel<<<grid, kThreads, kSmemBytes, stream>>>(mq, mk, mv, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

extern "C" int tx_flash_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int N,
                            int Kh, int Lq, int Lk, int head_dim, long long ldq, long long ldk, long long ldv,
                            long long ldo, int causal, float scale, int* status, cudaStream_t stream) {
  return tx_flash_fwd_seg(q, k, v, o, lse, B, N, Kh, Lq, Lk, head_dim, ldq, ldk, ldv, ldo, causal, scale, nullptr,
                          nullptr, status, stream);
}
