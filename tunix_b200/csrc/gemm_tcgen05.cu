// bf16 GEMM for sm_100a on the 5th-generation tensor cores.
//
//   C[M,N] (+)= alpha * A[M,K] * B[N,K]^T        (fp32 accumulation in TMEM)
//
// One persistent CTA per SM walks output tiles of 128 x BN (BN = 256, 128 or 64).
// Warp roles inside a CTA (192 threads):
//   warp 0     : TMA producer - one elected lane issues cp.async.bulk.tensor loads into a
//                ring of 128-byte-swizzled shared-memory stages.
//   warp 1     : owns TMEM allocation; one elected lane issues tcgen05.mma (UMMA 128xBNx16)
//                and tcgen05.commit to hand stages back / publish finished accumulators.
//   warps 2..5 : epilogue - tcgen05.ld the accumulator (one row per thread), scale,
//                optionally add the existing C, convert and store.
// Two accumulators live in TMEM (2 x BN columns), so the epilogue of tile i overlaps the
// main loop of tile i+1.
//
// Operand layouts. Either operand may be "K-major" (the reduction dimension is the
// contiguous one: A given as [M,K], B as [N,K]) or "MN-major" (A given as [K,M], B as
// [K,N]). That covers the three products of a linear layer without any transposes:
//   forward   y  = x  W^T   : A K-major,  B K-major
//   dgrad     dx = dy W     : A K-major,  B MN-major
//   wgrad     dW = dy^T x   : A MN-major, B MN-major
//
// No cluster launch and no multicast copies are used, so the kernel is safe to run in
// multi-GPU jobs, and its operands may live in peer memory.
#include "gemm_common.cuh"
#include "tx_host.h"

namespace {

using namespace tx;

constexpr int BM = 128;
constexpr int BK = 64;          // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int GROUP_M = 8;      // tile-order swizzle: 8 row-blocks share their B tiles in L2

template <int BN>
struct Cfg {
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : (BN == 64 ? 8 : 10));
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 256 /*barriers*/;
};

using txg::GemmParams;

__device__ __forceinline__ void tile_coords(int t, int mb, int nb, int& pm, int& pn) {
  txg::tile_coords(t, mb, nb, GROUP_M, pm, pn);
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_a2, const __grid_constant__ CUtensorMap map_b2,
                 const GemmParams p) {
  using C = Cfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle needs every stage 1024-byte aligned.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kStages * C::kStageBytes);
  // barrier layout: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * C::kStages;
  const uint32_t bar_tfull = bar_empty + 8 * C::kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int mb = (p.M + BM - 1) / BM;
  const int nb = (p.N + BN - 1) / BN;
  const int ks = p.k_splits > 1 ? p.k_splits : 1;
  const int num_tiles = mb * nb * ks;            // work items: (tile, K range)
  const int num_kb1 = (p.K + BK - 1) / BK;
  const int num_kb = num_kb1 + (p.K2 > 0 ? (p.K2 + BK - 1) / BK : 0);   // k-blocks of both operand pairs
  const int kb_per = (num_kb + ks - 1) / ks;     // the host picks ks so that no range is empty

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
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
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int pm, pn;
        tile_coords(t / ks, mb, nb, pm, pn);
        const int m0 = pm * BM, n0 = pn * BN;
        const int kb0 = (t % ks) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag)) {
            atomicOr(p.status, kStatusWaitTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t sa = smem_base + stage * C::kStageBytes;
          const uint32_t sb = sa + C::kABytes;
          mbar_expect_tx(full, C::kStageBytes);
          const bool second = kb >= num_kb1;                 // the low-rank pair follows the main pair
          const CUtensorMap* ma = second ? &map_a2 : &map_a;
          const CUtensorMap* mbp = second ? &map_b2 : &map_b;
          const int kc = (second ? kb - num_kb1 : kb) * BK;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i) tma_load_2d(sa + i * (BK * 128), ma, m0 + i * 64, kc, full);
          } else {
            tma_load_2d(sa, ma, kc, m0, full);
          }
          if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb + i * (BK * 128), mbp, n0 + i * 64, kc, full);
          } else {
            tma_load_2d(sb, mbp, kc, n0, full);
          }
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
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
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag)) {
          atomicOr(p.status, kStatusWaitTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        const int kb0 = (t % ks) * kb_per, kb1 = min(num_kb, kb0 + kb_per);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
            atomicOr(p.status, kStatusWaitTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * C::kStageBytes;
          const uint32_t sb = sa + C::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(sa + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(sa + k * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(sb + k * 2048, BK * 128, 1024)
                                     : make_smem_desc_sw128(sb + k * 32, 16, 1024);
            umma_bf16(tmem_d, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          umma_commit(bar_empty + 8 * stage);
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(bar_tfull + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int pm, pn;
      tile_coords(t / ks, mb, nb, pm, pn);
      const int row = pm * BM + quarter * 32 + lane;
      const int n0 = pn * BN;
      if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
        atomicOr(p.status, kStatusWaitTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        txg::store_row_chunk(p, row, n0 + c, r);
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // Teardown. On an aborted run give outstanding bulk copies a moment to land before the
  // shared memory is released.
  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

template <int BN, bool A_MN, bool B_MN>
int launch(const void* A, const void* B, const GemmParams& p, long long lda, long long ldb,
           cudaStream_t stream, int max_ctas, const void* A2 = nullptr, const void* B2 = nullptr, long long lda2 = 0,
           long long ldb2 = 0) {
  using C = Cfg<BN>;
  CUtensorMap ma, mbm;
  int rc;
  if (A_MN) rc = txh::make_map_2d_bf16(&ma, A, p.K, p.M, lda, BK, 64);
  else      rc = txh::make_map_2d_bf16(&ma, A, p.M, p.K, lda, BM, BK);
  if (rc) return 100 + rc;
  if (B_MN) rc = txh::make_map_2d_bf16(&mbm, B, p.K, p.N, ldb, BK, 64);
  else      rc = txh::make_map_2d_bf16(&mbm, B, p.N, p.K, ldb, BN, BK);
  if (rc) return 200 + rc;
  CUtensorMap ma2 = ma, mb2 = mbm;
  if (p.K2 > 0) {
    if (A_MN) rc = txh::make_map_2d_bf16(&ma2, A2, p.K2, p.M, lda2, BK, 64);
    else      rc = txh::make_map_2d_bf16(&ma2, A2, p.M, p.K2, lda2, BM, BK);
    if (rc) return 100 + rc;
    if (B_MN) rc = txh::make_map_2d_bf16(&mb2, B2, p.K2, p.N, ldb2, BK, 64);
    else      rc = txh::make_map_2d_bf16(&mb2, B2, p.N, p.K2, ldb2, BN, BK);
    if (rc) return 200 + rc;
  }
  static txh::DeviceFlag attr_flag;
  bool& attr_set = attr_flag.cur();
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN>;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess)
      return 300;
    attr_set = true;
  }
  const int mb = (p.M + BM - 1) / BM, nb = (p.N + BN - 1) / BN;
  int grid = mb * nb * (p.k_splits > 1 ? p.k_splits : 1);
  int sms = txh::sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (grid > sms) grid = sms;
  kern<<<grid, NUM_THREADS, C::kSmemBytes, stream>>>(ma, mbm, ma2, mb2, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

}  // namespace

// C ABI. a_mn / b_mn select the operand layout described at the top of this file:
//   a_mn == 0: A points at [M,K] (row stride lda);  a_mn == 1: A points at [K,M].
//   b_mn == 0: B points at [N,K] (row stride ldb);  b_mn == 1: B points at [K,N].
// Requirements: bf16 operands, 16-byte aligned bases, lda/ldb multiples of 8, N and ldc
// multiples of 8 (4 for fp32 C). `status` is a device int32 that receives error bits.
// `max_ctas` > 0 caps the grid (leaves SMs free for a concurrent copy/collective).
// Scratch of the split-K path: fp32 partial sums of one skinny GEMM at a time (M <= 128, M * N floats).
// One buffer per device; launches that use it must be ordered on one stream.
constexpr long long kSplitWsFloats = 128LL * 32768;
static __device__ __align__(256) float g_splitk_ws[kSplitWsFloats];

__global__ void splitk_finish_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ c, long long ldc,
                                     int M, int N) {
  const long long n4 = static_cast<long long>(M) * (N / 4);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(i / (N / 4)), q = static_cast<int>(i % (N / 4));
    const float4 v = reinterpret_cast<const float4*>(ws + static_cast<long long>(r) * N)[q];
    __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(c + static_cast<long long>(r) * ldc) + 2 * q;
    o[0] = __floats2bfloat162_rn(v.x, v.y);
    o[1] = __floats2bfloat162_rn(v.z, v.w);
  }
}

// The scratch address of the current device, looked up once per device (the lookup is not something to do
// inside a stream capture; `tx_gemm_warmup` lets callers force it early).
static float* splitk_workspace() {
  static float* cache[16] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  if (cache[dev] == nullptr) {
    float* ws = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ws), g_splitk_ws) != cudaSuccess) return nullptr;
    cache[dev] = ws;
  }
  return cache[dev];
}

extern "C" int tx_gemm_warmup() { return splitk_workspace() != nullptr ? 0 : 300; }

static int g_deterministic = 0;
// 1: no split-K (its partial sums meet through fp32 atomics, whose order varies from run to run); every product
// is then reduced in one fixed order and repeated launches give identical bits.
extern "C" void tx_gemm_set_deterministic(int v) { g_deterministic = v; }

// Policy of the general kernel for products with few rows (M <= 128; the decode path proper uses gemm_skinny.cu):
// 64-column tiles (32-column ones were measured slower on every decode shape but 4096 x 4096), and K split over
// several CTAs when fewer than 96 tiles exist.
constexpr int g_skinny_bn32 = 0;
constexpr int g_split_limit = 96;

static int g_disable_pair = 0;
// Test hook: 1 forces the single-CTA kernels for every shape.
extern "C" void tx_gemm_set_disable_pair(int v) { g_disable_pair = v; }

// C = alpha * (A B^T + A2 B2^T): the second pair (K2 columns, same layouts as the first; K2 == 0 for none)
// is accumulated in the same pass - fused low-rank adapters. lda2 / ldb2 multiples of 8.
extern "C" int tx_gemm_bf16_dual(const void* A, const void* B, const void* A2, const void* B2, void* C, int M, int N,
                                 int K, int K2, long long lda, long long ldb, long long lda2, long long ldb2,
                                 long long ldc, int a_mn, int b_mn, int c_fp32, int accumulate, float alpha,
                                 int* status, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || K2 < 0) return 1;
  if (K2 > 0 && (!A2 || !B2 || (lda2 & 7) || (ldb2 & 7) || (reinterpret_cast<uintptr_t>(A2) & 15) ||
                 (reinterpret_cast<uintptr_t>(B2) & 15)))
    return 2;
  if ((lda & 7) || (ldb & 7) || (N & 7) || (ldc & 3)) return 2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15))
    return 3;
  GemmParams p{C, ldc, M, N, K, c_fp32, accumulate, alpha, status, 1, K2, 0, {nullptr}};
  // Large problems: 256 x 256 tiles on CTA pairs (cta_group::2) halve the B traffic per SM.
  {
    const long long tiles_pair = static_cast<long long>((M + 255) / 256) * ((N + 255) / 256);
    const int pairs = txh::sm_count() / 2;
    if (!g_disable_pair && M >= 256 && N >= 256 && tiles_pair >= pairs)
      return tx_gemm_pair_launch(A, B, A2, B2, p, lda, ldb, lda2, ldb2, a_mn, b_mn, max_ctas, stream);
  }
  const int sel0 = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  // Skinny problems (decode: M <= 128 rows against a large weight) are bound by streaming B once.
  // Narrow 64-column tiles put 2-4x as many CTAs on that stream, which is what fills HBM.
  if (K2 == 0 && M <= BM && static_cast<long long>((N + 127) / 128) < 2LL * txh::sm_count()) {
    // Too few tiles to fill the GPU: split K over several CTAs per tile, sum the fp32 partials with
    // vector atomics in a scratch buffer, then round to bf16.
    const bool bn32 = g_skinny_bn32 && sel0 == 0;                // 32-column tiles: twice as many CTAs on the stream
    const int tiles = bn32 ? (N + 31) / 32 : (N + 63) / 64, num_kb = (K + BK - 1) / BK;
    int ks = tiles < g_split_limit ? (2 * txh::sm_count()) / tiles : 1;   // splitting only pays when few tiles exist
    if (ks > 8) ks = 8;
    if (ks > num_kb / 8) ks = num_kb / 8;
    if (g_deterministic) ks = 1;
    while (ks > 1 && (ks - 1) * ((num_kb + ks - 1) / ks) >= num_kb) --ks;     // no empty K range
    if (ks > 1 && !c_fp32 && !accumulate && (N & 3) == 0 && static_cast<long long>(M) * N <= kSplitWsFloats) {
      float* ws = splitk_workspace();
      if (ws == nullptr) return 300;
      if (cudaMemsetAsync(ws, 0, sizeof(float) * static_cast<size_t>(M) * N, stream) != cudaSuccess) return 400;
      GemmParams ps{ws, N, M, N, K, 1, 0, alpha, status, ks, 0, 0, {nullptr}};
      int rc;
      switch (sel0) {
        case 0: rc = bn32 ? launch<32, false, false>(A, B, ps, lda, ldb, stream, max_ctas)
                          : launch<64, false, false>(A, B, ps, lda, ldb, stream, max_ctas); break;
        case 1: rc = launch<64, false, true>(A, B, ps, lda, ldb, stream, max_ctas); break;
        case 2: rc = launch<64, true, false>(A, B, ps, lda, ldb, stream, max_ctas); break;
        default: rc = launch<64, true, true>(A, B, ps, lda, ldb, stream, max_ctas); break;
      }
      if (rc) return rc;
      const long long n4 = static_cast<long long>(M) * (N / 4);
      const int blocks = static_cast<int>(n4 / 256 + 1 < 592 ? n4 / 256 + 1 : 592);
      splitk_finish_kernel<<<blocks, 256, 0, stream>>>(ws, static_cast<__nv_bfloat16*>(C), ldc, M, N);
      return cudaGetLastError() == cudaSuccess ? 0 : 400;
    }
    switch (sel0) {
      case 0: return bn32 ? launch<32, false, false>(A, B, p, lda, ldb, stream, max_ctas)
                          : launch<64, false, false>(A, B, p, lda, ldb, stream, max_ctas);
      case 1: return launch<64, false, true>(A, B, p, lda, ldb, stream, max_ctas);
      case 2: return launch<64, true, false>(A, B, p, lda, ldb, stream, max_ctas);
      default: return launch<64, true, true>(A, B, p, lda, ldb, stream, max_ctas);
    }
  }
  // Wide tiles unless that would leave most SMs idle.
  const long long tiles256 = static_cast<long long>((M + BM - 1) / BM) * ((N + 255) / 256);
  const bool bn256 = tiles256 >= txh::sm_count() || (N % 256 == 0 && tiles256 * 2 > 3 * txh::sm_count());
  const int sel = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  if (bn256 || tiles256 >= 96) {
    switch (sel) {
      case 0: return launch<256, false, false>(A, B, p, lda, ldb, stream, max_ctas, A2, B2, lda2, ldb2);
      case 1: return launch<256, false, true>(A, B, p, lda, ldb, stream, max_ctas, A2, B2, lda2, ldb2);
      case 2: return launch<256, true, false>(A, B, p, lda, ldb, stream, max_ctas, A2, B2, lda2, ldb2);
      default: return launch<256, true, true>(A, B, p, lda, ldb, stream, max_ctas, A2, B2, lda2, ldb2);
    }
  }
  switch (sel) {
    case 0: return launch<128, false, false>(A, B, p, lda, ldb, stream, max_ctas, A2, B2, lda2, ldb2);
    case 1: return launch<128, false, true>(A, B, p, lda, ldb, stream, max_ctas, A2, B2, lda2, ldb2);
    case 2: return launch<128, true, false>(A, B, p, lda, ldb, stream, max_ctas, A2, B2, lda2, ldb2);
    default: return launch<128, true, true>(A, B, p, lda, ldb, stream, max_ctas, A2, B2, lda2, ldb2);
  }
}

extern "C" int tx_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                            long long ldb, long long ldc, int a_mn, int b_mn, int c_fp32, int accumulate,
                            float alpha, int* status, int max_ctas, cudaStream_t stream) {
  return tx_gemm_bf16_dual(A, B, nullptr, nullptr, C, M, N, K, 0, lda, ldb, 0, 0, ldc, a_mn, b_mn, c_fp32, accumulate,
                           alpha, status, max_ctas, stream);
}

// Rounds a fp32 [M, N] sum buffer (row stride N) to bf16 C (row stride ldc). N a multiple of 4.
extern "C" int tx_f32_sum_to_bf16(const float* ws, void* C, long long ldc, int M, int N, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (N & 3) return 1;
  const long long n4 = static_cast<long long>(M) * (N / 4);
  const int blocks = static_cast<int>(n4 / 256 + 1 < 592 ? n4 / 256 + 1 : 592);
  splitk_finish_kernel<<<blocks, 256, 0, stream>>>(ws, static_cast<__nv_bfloat16*>(C), ldc, M, N);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

// Row-parallel linear of a tensor-parallel group with the all-reduce fused into the GEMM epilogue:
// every rank computes its partial product A B^T (its shard of K) and adds each output tile, with fp32 vector
// atomics over NVLink, into the zero-filled [M, N] fp32 buffer of every rank (`dst[i]`, i < n_peers, peer-mapped
// pointers, own buffer included). Once all ranks' kernels have finished (a barrier the caller provides) every
// buffer holds the full sum. Plain peer stores only: no multicast. M x N x K in the caller's usual layouts.
extern "C" int tx_gemm_bf16_allreduce(const void* A, const void* B, void* const* dst, int n_peers, int M, int N, int K,
                                      long long lda, long long ldb, int a_mn, int b_mn, float alpha, int* status,
                                      cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || n_peers < 1 || n_peers > 8 || !dst) return 1;
  if ((lda & 7) || (ldb & 7) || (N & 7)) return 2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return 3;
  GemmParams p{nullptr, N, M, N, K, 1, 0, alpha, status, 1, 0, n_peers, {nullptr}};
  for (int i = 0; i < n_peers; ++i) {
    if (!dst[i] || (reinterpret_cast<uintptr_t>(dst[i]) & 15)) return 3;
    p.red_dst[i] = static_cast<float*>(dst[i]);
  }
  const int sel = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  if (M <= BM) {
    switch (sel) {
      case 0: return launch<64, false, false>(A, B, p, lda, ldb, stream, 0);
      case 1: return launch<64, false, true>(A, B, p, lda, ldb, stream, 0);
      case 2: return launch<64, true, false>(A, B, p, lda, ldb, stream, 0);
      default: return launch<64, true, true>(A, B, p, lda, ldb, stream, 0);
    }
  }
  switch (sel) {
    case 0: return launch<256, false, false>(A, B, p, lda, ldb, stream, 0);
    case 1: return launch<256, false, true>(A, B, p, lda, ldb, stream, 0);
    case 2: return launch<256, true, false>(A, B, p, lda, ldb, stream, 0);
    default: return launch<256, true, true>(A, B, p, lda, ldb, stream, 0);
  }
}
