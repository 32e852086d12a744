// bf16 GEMM on CTA pairs: tcgen05.mma.cta_group::2, one 256 x 256 output tile per pair.
//
// Two CTAs on neighbouring SMs form a cluster. Each stages its own half of the tile's operands -
// 128 rows of A and 128 of the 256 B rows (N) - so per SM and k-block 32 KB arrive from L2 for
// 128 x 256 x 64 MACs, two thirds of what the single-CTA 128 x 256 tile needs; at 148 SMs the
// L2 -> shared-memory traffic is what limits the single-CTA kernel. The leader CTA (cluster
// rank 0) issues the MMAs, which read both CTAs' shared memory and write 128 accumulator rows
// into each CTA's TMEM. Each CTA drains its own TMEM half in its epilogue warps.
//
// Synchronisation (all mbarriers, all waits bounded):
//   full[s]    leader only. The leader's producer arms it with the bytes of BOTH CTAs; both
//              CTAs' TMA loads complete on it (cta_group::2 loads may signal the peer's barrier).
//   empty[s]   one per CTA; tcgen05.commit multicast to both when the MMAs reading stage s retire.
//   tfull[a]   one per CTA; commit multicast when accumulator a is complete.
//   tempty[a]  leader only; one arrival per epilogue warp of either CTA (8) once a is drained.
// No TMA load uses cluster multicast: every CTA fetches its own operand half.
#include "gemm_common.cuh"
#include "tx_host.h"

namespace {

using namespace tx;
using txg::GemmParams;

constexpr int BM_CTA = 128;     // rows of A (and accumulator rows) per CTA
constexpr int BN = 256;         // tile width; each CTA stages BN / 2 rows of B
constexpr int BN_CTA = BN / 2;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 8;
constexpr int kStages = 6;
constexpr int kABytes = BM_CTA * BK * 2;      // 16 KB
constexpr int kBBytes = BN_CTA * BK * 2;      // 16 KB
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 2 * BN;             // two accumulators
constexpr int kRedBytes = 32 * 128;            // one [32 rows x 32 fp32] swizzled box
constexpr int kRedBufBytes = 4 * 2 * kRedBytes; // per epilogue warp: two boxes (double buffer)
constexpr int kSmemBytes = kStages * kStageBytes + kRedBufBytes + 1024 + 256;

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
                      const __grid_constant__ CUtensorMap map_c, const GemmParams p, const int red_epilogue) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t red_base = smem_base + kStages * kStageBytes;      // 1024-byte aligned
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + kStages * kStageBytes + kRedBufBytes);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_tfull = bar_empty + 8 * kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();          // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  const int mb = (p.M + 2 * BM_CTA - 1) / (2 * BM_CTA);
  const int nb = (p.N + BN - 1) / BN;
  const int num_tiles = mb * nb;
  const int num_kb1 = (p.K + BK - 1) / BK;
  const int num_kb = num_kb1 + (p.K2 > 0 ? (p.K2 + BK - 1) / BK : 0);   // k-blocks of both operand pairs

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 8);
    }
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();       // the peer's barriers are initialised before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        int pm, pn;
        txg::tile_coords(t, mb, nb, GROUP_M, pm, pn);
        const int m0 = pm * 2 * BM_CTA + cta * BM_CTA;
        const int n0 = pn * BN + cta * BN_CTA;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag)) {
            atomicOr(p.status, kStatusWaitTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t full_leader = map_to_cta(bar_full + 8 * stage, 0);
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
          if (cta == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * kStageBytes);
          const bool second = kb >= num_kb1;                 // the low-rank pair follows the main pair
          const CUtensorMap* ma = second ? &map_a2 : &map_a;
          const CUtensorMap* mbp = second ? &map_b2 : &map_b;
          const int kc = (second ? kb - num_kb1 : kb) * BK;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BM_CTA / 64; ++i)
              tma_load_2d_pair(sa + i * (BK * 128), ma, m0 + i * 64, kc, full_leader);
          } else {
            tma_load_2d_pair(sa, ma, kc, m0, full_leader);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN_CTA / 64; ++i)
              tma_load_2d_pair(sb + i * (BK * 128), mbp, n0 + i * 64, kc, full_leader);
          } else {
            tma_load_2d_pair(sb, mbp, kc, n0, full_leader);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (cta == 0 && elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * BM_CTA, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag)) {
          atomicOr(p.status, kStatusWaitTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
            atomicOr(p.status, kStatusWaitTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_bf16_pair(tmem_d, da, db, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(bar_empty + 8 * stage, 3);     // both CTAs may refill this stage
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit_pair(bar_tfull + 8 * acc, 3);         // both CTAs may drain this accumulator
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int quarter = warp & 3;
    const uint32_t tempty_leader0 = map_to_cta(bar_tempty, 0);
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      int pm, pn;
      txg::tile_coords(t, mb, nb, GROUP_M, pm, pn);
      const int row = pm * 2 * BM_CTA + cta * BM_CTA + quarter * 32 + lane;
      const int n0 = pn * BN;
      if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
        atomicOr(p.status, kStatusWaitTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if (red_epilogue) {
        // fp32 C += tile: each warp stages a [32 x 32] box in shared memory (128-byte swizzle) and hands it
        // to the TMA unit as a reduce-add, so C is never read into the SM and the adds run in L2.
        const int row0 = pm * 2 * BM_CTA + cta * BM_CTA + quarter * 32;
        const uint32_t my_red = red_base + quarter * (2 * kRedBytes);
        uint8_t* my_red_gen = smem_gen + kStages * kStageBytes + quarter * (2 * kRedBytes);
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          const int buf = (c >> 5) & 1;
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c, r);
          tmem_ld_wait();
          if (lane == 0) tma_store_wait_read<1>();      // the box issued two chunks ago has been read
          __syncwarp();
          uint8_t* rowp = my_red_gen + buf * kRedBytes + lane * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 v = make_float4(__uint_as_float(r[4 * j]) * p.alpha, __uint_as_float(r[4 * j + 1]) * p.alpha,
                                         __uint_as_float(r[4 * j + 2]) * p.alpha,
                                         __uint_as_float(r[4 * j + 3]) * p.alpha);
            *reinterpret_cast<float4*>(rowp + ((j ^ (lane & 7)) << 4)) = v;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < p.M && n0 + c < p.N) {
            tma_reduce_add_2d(&map_c, my_red + buf * kRedBytes, n0 + c, row0);
            tma_store_commit();
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c, r);
          tmem_ld_wait();
          txg::store_row_chunk(p, row, n0 + c, r);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(tempty_leader0 + 8 * acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (red_epilogue && lane == 0) tma_store_wait<0>();   // every reduce has landed before shared memory goes away
  }

  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();       // nobody leaves while the peer may still touch its memory or barriers
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <bool A_MN, bool B_MN>
int launch(const void* A, const void* B, const void* A2, const void* B2, const GemmParams& p, long long lda,
           long long ldb, long long lda2, long long ldb2, int max_ctas, cudaStream_t stream) {
  CUtensorMap ma, mbm;
  int rc;
  if (A_MN) rc = txh::make_map_2d_bf16(&ma, A, p.K, p.M, lda, BK, 64);
  else      rc = txh::make_map_2d_bf16(&ma, A, p.M, p.K, lda, BM_CTA, BK);
  if (rc) return 100 + rc;
  if (B_MN) rc = txh::make_map_2d_bf16(&mbm, B, p.K, p.N, ldb, BK, 64);
  else      rc = txh::make_map_2d_bf16(&mbm, B, p.N, p.K, ldb, BN_CTA, BK);
  if (rc) return 200 + rc;
  CUtensorMap ma2 = ma, mb2 = mbm;
  if (p.K2 > 0) {
    if (A_MN) rc = txh::make_map_2d_bf16(&ma2, A2, p.K2, p.M, lda2, BK, 64);
    else      rc = txh::make_map_2d_bf16(&ma2, A2, p.M, p.K2, lda2, BM_CTA, BK);
    if (rc) return 100 + rc;
    if (B_MN) rc = txh::make_map_2d_bf16(&mb2, B2, p.K2, p.N, ldb2, BK, 64);
    else      rc = txh::make_map_2d_bf16(&mb2, B2, p.N, p.K2, ldb2, BN_CTA, BK);
    if (rc) return 200 + rc;
  }
  // fp32 accumulation into C (gradient accumulation of weight gradients) goes through TMA reduce-add.
  CUtensorMap mc = ma;
  int red = 0;
  if (p.c_fp32 && p.accumulate && p.ldc % 4 == 0 && reinterpret_cast<uintptr_t>(p.C) % 16 == 0) {
    if (txh::make_map_2d_f32(&mc, p.C, p.M, p.N, p.ldc, 32) == 0) red = 1;
    else mc = ma;
  }
  auto kern = gemm_bf16_pair_kernel<A_MN, B_MN>;
  static txh::DeviceFlag attr_flag;
  bool& attr_set = attr_flag.cur();
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) return 300;
    attr_set = true;
  }
  const int mb = (p.M + 2 * BM_CTA - 1) / (2 * BM_CTA), nb = (p.N + BN - 1) / BN;
  int sms = txh::sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  int pairs = mb * nb;
  if (pairs > sms / 2) pairs = sms / 2;
  if (pairs < 1) pairs = 1;
  kern<<<2 * pairs, NUM_THREADS, kSmemBytes, stream>>>(ma, mbm, ma2, mb2, mc, p, red);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

}  // namespace

int tx_gemm_pair_launch(const void* A, const void* B, const void* A2, const void* B2, const txg::GemmParams& p,
                        long long lda, long long ldb, long long lda2, long long ldb2, int a_mn, int b_mn, int max_ctas,
                        cudaStream_t stream) {
  const int sel = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  switch (sel) {
    case 0: return launch<false, false>(A, B, A2, B2, p, lda, ldb, lda2, ldb2, max_ctas, stream);
    case 1: return launch<false, true>(A, B, A2, B2, p, lda, ldb, lda2, ldb2, max_ctas, stream);
    case 2: return launch<true, false>(A, B, A2, B2, p, lda, ldb, lda2, ldb2, max_ctas, stream);
    default: return launch<true, true>(A, B, A2, B2, p, lda, ldb, lda2, ldb2, max_ctas, stream);
  }
}
