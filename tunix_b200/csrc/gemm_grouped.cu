// Grouped bf16 GEMM for mixture-of-experts layers on the sm_100a tensor cores: one launch
// covers every expert, and the kernel reads which rows belong to which expert from device
// memory, so the host never waits for the routing result.
//
// Row layout. The rows routed to the experts are stored expert by expert, each expert's
// block padded with zero rows to a multiple of 128, so a 128-row tile never straddles two
// experts:
//   offsets[e]      first row of expert e (int32, E + 1 entries, multiples of 128)
//   tile_expert[i]  expert of row tile i (rows [128 i, 128 i + 128)), or -1 past the last block
// With W = [E, N, K] stacked expert weights:
//   mode 0  forward  Y [R, N]   = X [R, K]  W[e]^T    (e = expert of the row tile)
//   mode 1  dgrad    dX [R, K]  = dY [R, N] W[e]
//   mode 2  wgrad    dW[e][N,K] (+)= dY[rows of e, N]^T X[rows of e, K]
// Modes 0/1 skip tiles whose tile_expert is -1 (their output rows are left untouched); mode 2
// skips experts without rows (their dW is left untouched: zero it first unless accumulating).
//
// Same structure as the dense kernel (gemm_tcgen05.cu): persistent CTAs of 192 threads, warp 0
// = TMA producer, warp 1 = tcgen05.mma issuer with two TMEM accumulators, warps 2..5 =
// epilogue; tiles of 128 x 128, 6 shared-memory stages. No cluster launch, no multicast.
#include "gemm_common.cuh"
#include "tx_host.h"

namespace {

using namespace tx;
using txg::GemmParams;

constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int kStages = 6;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BN * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kTmemCols = 2 * BN;
constexpr int kRedBytes = 32 * 128;             // one [32 rows x 32 fp32] swizzled box of the reduce-add epilogue
constexpr int kRedBufBytes = 4 * 2 * kRedBytes; // per epilogue warp: two boxes (double buffer)
constexpr int kSmemBytes = kStages * kStageBytes + kRedBufBytes + 1024 + 256;

struct GroupedParams {
  GemmParams g;            // C, ldc, M/N/K = extents of the tile grid and of the reduction (modes 0/1)
  const int* tile_expert;  // modes 0/1
  const int* offsets;      // mode 2
  int num_experts;
  int estride;             // rows per expert in the stacked operand (B in modes 0/1, C in mode 2)
  int red_epilogue;        // mode 2 with fp32 accumulation: C += tile through TMA reduce-adds (C is never read)
};

// One unit of work: an output tile and the K range that produces it.
struct Item {
  int m0, n0;        // tile origin inside the tile grid
  int b_row;         // row offset of this expert inside the stacked B operand
  int c_row;         // row offset of this expert inside C (mode 2)
  int kb0, kb1;      // k-blocks [kb0, kb1) of 64
};

template <int MODE>
__device__ __forceinline__ bool decode_item(const GroupedParams& p, int t, int mb, int nb, Item& it) {
  if (MODE == 2) {
    const int per = mb * nb;
    const int e = t / per, r = t - e * per;
    it.m0 = (r % mb) * BM;
    it.n0 = (r / mb) * BN;
    it.b_row = 0;
    it.c_row = e * p.estride;
    it.kb0 = __ldg(p.offsets + e) / BK;
    it.kb1 = __ldg(p.offsets + e + 1) / BK;
    return it.kb1 > it.kb0;
  }
  int pm, pn;
  txg::tile_coords(t, mb, nb, 8, pm, pn);
  const int e = __ldg(p.tile_expert + pm);
  if (e < 0 || e >= p.num_experts) return false;
  it.m0 = pm * BM;
  it.n0 = pn * BN;
  it.b_row = e * p.estride;
  it.c_row = 0;
  it.kb0 = 0;
  it.kb1 = (p.g.K + BK - 1) / BK;
  return true;
}

template <bool A_MN, bool B_MN, int MODE>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_grouped_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ CUtensorMap map_c, const GroupedParams p) {
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
  const int mb = (p.g.M + BM - 1) / BM;
  const int nb = (p.g.N + BN - 1) / BN;
  const int num_items = (MODE == 2 ? p.num_experts : 1) * mb * nb;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 128);
    }
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

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_items && ok; t += gridDim.x) {
        Item it;
        if (!decode_item<MODE>(p, t, mb, nb, it)) continue;
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag)) {
            atomicOr(p.g.status, kStatusWaitTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
          mbar_expect_tx(full, kStageBytes);
          const int kc = kb * BK;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * (BK * 128), &map_a, it.m0 + i * 64, kc, full);
          } else {
            tma_load_2d(sa, &map_a, kc, it.m0, full);
          }
          if (B_MN) {
            // modes 1 and 2: the reduction index is the row of B; mode 1 adds the expert's row offset
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(sb + i * (BK * 128), &map_b, it.n0 + i * 64, kc + it.b_row, full);
          } else {
            tma_load_2d(sb, &map_b, kc, it.n0 + it.b_row, full);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_items && ok; t += gridDim.x) {
        Item it;
        if (!decode_item<MODE>(p, t, mb, nb, it)) continue;
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag)) {
          atomicOr(p.g.status, kStatusWaitTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = it.kb0; kb < it.kb1; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
            atomicOr(p.g.status, kStatusWaitTimeoutMma);
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
            umma_bf16(tmem_d, da, db, idesc, (kb > it.kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty + 8 * stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(bar_tfull + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    GemmParams g = p.g;
    if (MODE == 2) g.M = p.num_experts * p.estride;       // C is the stack of all experts' [M, N] blocks
    for (int t = blockIdx.x; t < num_items; t += gridDim.x) {
      Item it;
      if (!decode_item<MODE>(p, t, mb, nb, it)) continue;
      const int local_row = it.m0 + quarter * 32 + lane;
      if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
        atomicOr(p.g.status, kStatusWaitTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if (MODE == 2 && p.red_epilogue) {
        // each warp stages [32 x 32] fp32 boxes (128-byte swizzle) and hands them to the TMA unit as reduce-adds:
        // coalesced, and the adds run in L2. A warp's 32 rows lie inside one expert (M is a multiple of 32).
        const int row0 = it.m0 + quarter * 32;
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
            const float4 v = make_float4(__uint_as_float(r[4 * j]) * p.g.alpha, __uint_as_float(r[4 * j + 1]) * p.g.alpha,
                                         __uint_as_float(r[4 * j + 2]) * p.g.alpha,
                                         __uint_as_float(r[4 * j + 3]) * p.g.alpha);
            *reinterpret_cast<float4*>(rowp + ((j ^ (lane & 7)) << 4)) = v;
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row0 < p.g.M && it.n0 + c < p.g.N) {
            tma_reduce_add_2d(&map_c, my_red + buf * kRedBytes, it.n0 + c, it.c_row + row0);
            tma_store_commit();
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr + c, r);
          tmem_ld_wait();
          if (local_row < p.g.M) txg::store_row_chunk(g, it.c_row + local_row, it.n0 + c, r);
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
    if (MODE == 2 && p.red_epilogue && lane == 0) tma_store_wait<0>();   // reduces have landed before smem goes away
  }

  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <bool A_MN, bool B_MN, int MODE>
int launch(const CUtensorMap& ma, const CUtensorMap& mbm, const CUtensorMap& mc, const GroupedParams& p,
           cudaStream_t stream) {
  static txh::DeviceFlag attr_flag;
  bool& attr_set = attr_flag.cur();
  auto kern = gemm_grouped_kernel<A_MN, B_MN, MODE>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess)
      return 300;
    attr_set = true;
  }
  const long long mb = (p.g.M + BM - 1) / BM, nb = (p.g.N + BN - 1) / BN;
  long long items = (MODE == 2 ? p.num_experts : 1) * mb * nb;
  int grid = static_cast<int>(items < txh::sm_count() ? items : txh::sm_count());
  kern<<<grid, NUM_THREADS, kSmemBytes, stream>>>(ma, mbm, mc, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

}  // namespace

// C ABI. W is the stack [E, N, K] of expert weights (row stride ldw); R is the padded row count
// (a multiple of 128). Shapes by mode are given at the top of this file:
//   mode 0: A = X [R, K],  B = W,        C = Y  [R, N]
//   mode 1: A = dY [R, N], B = W,        C = dX [R, K]
//   mode 2: A = dY [R, N], B = X [R, K], C = dW [E * N, K]   (c_fp32 / accumulate as in the dense GEMM)
// N and K multiples of 8 (N a multiple of 64 in mode 1); bases 16-byte aligned; lda/ldb multiples of 8.
extern "C" int tx_gemm_grouped_bf16(const void* A, const void* B, void* C, const int* tile_expert, const int* offsets,
                                    int mode, int R, int N, int K, int E, long long lda, long long ldb,
                                    long long ldc, int c_fp32, int accumulate, float alpha, int* status,
                                    cudaStream_t stream) {
  if (R <= 0 || N <= 0 || K <= 0 || E <= 0 || mode < 0 || mode > 2) return 1;
  if ((R & 127) || (N & 7) || (K & 7) || (lda & 7) || (ldb & 7) || (ldc & 3)) return 2;
  if (mode == 1 && (N & 63)) return 2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15))
    return 3;
  if ((mode == 2 && !offsets) || (mode != 2 && !tile_expert)) return 1;
  CUtensorMap ma, mbm;
  GroupedParams p{};
  p.g = GemmParams{C, ldc, 0, 0, 0, c_fp32, accumulate, alpha, status, 1, 0, 0, {nullptr}};
  p.tile_expert = tile_expert;
  p.offsets = offsets;
  p.num_experts = E;
  int rc;
  if (mode == 0) {
    p.g.M = R; p.g.N = N; p.g.K = K; p.estride = N;
    rc = txh::make_map_2d_bf16(&ma, A, R, K, lda, BM, BK);
    if (rc) return 100 + rc;
    rc = txh::make_map_2d_bf16(&mbm, B, static_cast<uint64_t>(E) * N, K, ldb, BN, BK);
    if (rc) return 200 + rc;
    return launch<false, false, 0>(ma, mbm, ma, p, stream);
  }
  if (mode == 1) {
    p.g.M = R; p.g.N = K; p.g.K = N; p.estride = N;
    rc = txh::make_map_2d_bf16(&ma, A, R, N, lda, BM, BK);
    if (rc) return 100 + rc;
    rc = txh::make_map_2d_bf16(&mbm, B, static_cast<uint64_t>(E) * N, K, ldb, BK, 64);
    if (rc) return 200 + rc;
    return launch<false, true, 1>(ma, mbm, ma, p, stream);
  }
  p.g.M = N; p.g.N = K; p.g.K = 0; p.estride = N;
  rc = txh::make_map_2d_bf16(&ma, A, R, N, lda, BK, 64);
  if (rc) return 100 + rc;
  rc = txh::make_map_2d_bf16(&mbm, B, R, K, ldb, BK, 64);
  if (rc) return 200 + rc;
  CUtensorMap mc = ma;
  if (c_fp32 && accumulate && (N % 32) == 0) {
    rc = txh::make_map_2d_f32(&mc, C, static_cast<uint64_t>(E) * N, K, ldc, 32);
    if (rc) return 300 + rc;
    p.red_epilogue = 1;
  }
  return launch<true, true, 2>(ma, mbm, mc, p, stream);
}
