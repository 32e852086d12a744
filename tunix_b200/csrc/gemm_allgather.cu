// All-gather fused into its consuming GEMM (sharded weights over NVLink peer memory):
//
//   C[M, N] = A[M, K] * W[N, K]^T     with W row-sharded over `world` ranks: rank r holds W[r N/world : (r+1) N/world]
//
// No separate all-gather runs and the full W is never needed before the kernel starts. One launch does both:
//   * warps 6..9 of every CTA are copy warps. Together, all CTAs pull the remote shards one "slab" (256 or 128
//     rows = one column of output tiles) at a time with plain 16-byte peer loads into a local staging buffer; every CTA
//     copies its 1/grid share of EACH slab, so slabs complete one after another at the full link rate, in the
//     order in which the tensor-core side will need them. A per-slab counter in global memory counts the CTAs
//     that have finished their share.
//   * warp 0 (TMA producer), warp 1 (tcgen05.mma issuer) and warps 2..5 (epilogue) are the persistent GEMM of
//     gemm_tcgen05.cu with 128 x 256 (or 128 x 128) tiles. Tiles are walked slab by slab starting with this rank's OWN rows
//     (read in place, no copy, no wait), then the next rank's, and so on around the ring, so each rank starts on
//     a different peer. Before the first TMA load of a remote slab the producer waits (bounded) until the slab's
//     counter has reached the grid size.
// The copy never waits for anything, so there is no circular dependency; a producer wait that runs out sets
// status bit 16 and the CTA drains. Plain peer loads only: no multicast, no TMA from peer memory.
#include "gemm_common.cuh"
#include "tx_host.h"

namespace {

using namespace tx;
using txg::GemmParams;

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 320;
constexpr int COPY_THREADS = 128;
constexpr int kABytes = BM * BK * 2;
constexpr int kMaxPeers = 8;

// Tile width BN = slab height: 256 (4 stages of 48 KB, both TMEM accumulators fill the 512 columns) when the
// shards divide into 256-row slabs, else 128 (6 stages of 32 KB).
template <int BN>
struct Cfg {
  static constexpr int kStages = BN == 256 ? 4 : 6;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

struct GatherParams {
  GemmParams g;
  const __nv_bfloat16* shard[kMaxPeers];   // rank r's rows [r N/world, (r+1) N/world), row stride ldb (peer-mapped)
  long long ldb;
  __nv_bfloat16* stage;                    // [N, K] local staging, row stride K
  int* slab_count;                         // [N / 128], zeroed before the launch
  int world, rank;
  unsigned long long wait_limit_ns;
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_allgather_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_own,
                      const __grid_constant__ CUtensorMap map_stage, const GatherParams p) {
  constexpr int kStages = Cfg<BN>::kStages;
  constexpr int kStageBytes = Cfg<BN>::kStageBytes;
  constexpr int kTmemCols = Cfg<BN>::kTmemCols;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + kStages * kStageBytes);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kStages;
  const uint32_t bar_tfull = bar_empty + 8 * kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int mb = (p.g.M + BM - 1) / BM;
  const int n_slabs = p.g.N / BN;
  const int per_rank = n_slabs / p.world;            // slabs owned by each rank
  const int num_tiles = mb * n_slabs;
  const int num_kb = (p.g.K + BK - 1) / BK;
  const int own_first = p.rank * per_rank;

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

  // tile t -> (row block, slab): slab-major, own slabs first, then around the ring of ranks
  auto tile_of = [&](int t, int& pm, int& slab) {
    const int order = t / mb;
    pm = t - order * mb;
    slab = own_first + order;
    if (slab >= n_slabs) slab -= n_slabs;
  };

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_own);
      tma_prefetch_desc(&map_stage);
      int stage = 0;
      uint32_t phase = 0;
      int ready_slab = -1;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int pm, slab;
        tile_of(t, pm, slab);
        const bool own = slab >= own_first && slab < own_first + per_rank;
        if (!own && slab != ready_slab) {
          const uint64_t t0 = globaltimer_ns();
          while (ld_acquire_gpu(p.slab_count + slab) < static_cast<int>(gridDim.x)) {
            if (*abort_flag || globaltimer_ns() - t0 > p.wait_limit_ns) {
              *abort_flag = 1;
              atomicOr(p.g.status, kStatusPeerWaitTimeout);
              ok = false;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) break;
          fence_proxy_async_all();          // the staged rows were written by ordinary stores; TMA reads them
          ready_slab = slab;
        }
        const CUtensorMap* mbp = own ? &map_own : &map_stage;
        const int brow = own ? (slab - own_first) * BN : slab * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag)) {
            atomicOr(p.g.status, kStatusWaitTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t sa = smem_base + stage * kStageBytes;
          mbar_expect_tx(full, kStageBytes);
          tma_load_2d(sa, &map_a, kb * BK, pm * BM, full);
          tma_load_2d(sa + kABytes, mbp, kb * BK, brow, full);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag)) {
          atomicOr(p.g.status, kStatusWaitTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
            atomicOr(p.g.status, kStatusWaitTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * kStageBytes;
          const uint32_t sb = sa + kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_bf16(tmem_d, make_smem_desc_sw128(sa + k * 32, 16, 1024), make_smem_desc_sw128(sb + k * 32, 16, 1024),
                      idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(bar_empty + 8 * stage);
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(bar_tfull + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      int pm, slab;
      tile_of(t, pm, slab);
      const int row = pm * BM + quarter * 32 + lane;
      if (!mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag)) {
        atomicOr(p.g.status, kStatusWaitTimeoutEpilogue);
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr + c, r);
        tmem_ld_wait();
        txg::store_row_chunk(p.g, row, slab * BN + c, r);
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  } else {
    // ------------------------------------------------------------ copy warps (6..9): the all-gather
    const int ct = threadIdx.x - 6 * 32;                 // 0..127
    const int k8 = p.g.K / 8;                            // 16-byte chunks per row
    const long long chunks = static_cast<long long>(BN) * k8;
    for (int order = per_rank; order < n_slabs; ++order) {
      int slab = own_first + order;
      if (slab >= n_slabs) slab -= n_slabs;
      const int owner = slab / per_rank;
      const __nv_bfloat16* src = p.shard[owner] + static_cast<long long>(slab - owner * per_rank) * BN * p.ldb;
      __nv_bfloat16* dst = p.stage + static_cast<long long>(slab) * BN * p.g.K;
      const long long step = static_cast<long long>(gridDim.x) * COPY_THREADS;
      long long c = static_cast<long long>(blockIdx.x) * COPY_THREADS + ct;
      // four independent 16-byte peer loads in flight per thread
      for (; c + 3 * step < chunks; c += 4 * step) {
        uint4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const long long cc = c + u * step;
          v[u] = *reinterpret_cast<const uint4*>(src + (cc / k8) * p.ldb + (cc % k8) * 8);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const long long cc = c + u * step;
          *reinterpret_cast<uint4*>(dst + (cc / k8) * p.g.K + (cc % k8) * 8) = v[u];
        }
      }
      for (; c < chunks; c += step)
        *reinterpret_cast<uint4*>(dst + (c / k8) * p.g.K + (c % k8) * 8) =
            *reinterpret_cast<const uint4*>(src + (c / k8) * p.ldb + (c % k8) * 8);
      fence_proxy_async_all();
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");     // the four copy warps only; nothing external is awaited
      if (ct == 0) atomicAdd(p.slab_count + slab, 1);
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

// shards[r]: rank r's rows of W (bf16, row stride ldb), peer-mapped; shards[rank] is local. stage: local [N, K] bf16
// scratch; slab_count: local int32 [N / 128] scratch (N / 256 entries are used with 256-row slabs) (this call zeroes it on `stream`). A [M, K] (stride lda),
// C [M, N] bf16 or fp32 (stride ldc). Needs N % (128 * world) == 0, K % 64 == 0, world <= 8.
// Every rank of the group must have finished writing its shard before any rank launches (a barrier the caller
// provides), and must not overwrite it before all ranks' kernels have finished.
template <int BN>
static int launch_gather(const void* A, void* const* shards, void* stage, GatherParams& p, int M, int N, int K,
                         long long lda, long long ldb, int world, int rank, cudaStream_t stream) {
  CUtensorMap ma, mown, mstage;
  int rc = txh::make_map_2d_bf16(&ma, A, M, K, lda, BM, BK);
  if (rc) return 100 + rc;
  rc = txh::make_map_2d_bf16(&mown, shards[rank], N / world, K, ldb, BN, BK);
  if (rc) return 200 + rc;
  rc = txh::make_map_2d_bf16(&mstage, stage, N, K, K, BN, BK);
  if (rc) return 200 + rc;
  static txh::DeviceFlag attr_flag;
  bool& attr_set = attr_flag.cur();
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_allgather_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Cfg<BN>::kSmemBytes) != cudaSuccess)
      return 300;
    attr_set = true;
  }
  if (cudaMemsetAsync(p.slab_count, 0, sizeof(int) * (N / BN), stream) != cudaSuccess) return 400;
  const long long tiles = static_cast<long long>((M + BM - 1) / BM) * (N / BN);
  const int grid = static_cast<int>(tiles < txh::sm_count() ? tiles : txh::sm_count());
  gemm_allgather_kernel<BN><<<grid, NUM_THREADS, Cfg<BN>::kSmemBytes, stream>>>(ma, mown, mstage, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

extern "C" int tx_gemm_bf16_allgather_b(const void* A, void* const* shards, int world, int rank, void* stage,
                                        int* slab_count, void* C, int M, int N, int K, long long lda, long long ldb,
                                        long long ldc, int c_fp32, int accumulate, float alpha, long long wait_limit_ms,
                                        int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return 1;
  if ((N % (128 * world)) || (K % BK) || (lda & 7) || (ldb & 7) || (ldc & 3)) return 2;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(C) & 15) ||
      (reinterpret_cast<uintptr_t>(stage) & 15))
    return 3;
  GatherParams p{};
  p.g = GemmParams{C, ldc, M, N, K, c_fp32, accumulate, alpha, status, 1, 0, 0, {nullptr}};
  for (int i = 0; i < world; ++i) {
    if (!shards[i] || (reinterpret_cast<uintptr_t>(shards[i]) & 15)) return 3;
    p.shard[i] = static_cast<const __nv_bfloat16*>(shards[i]);
  }
  p.ldb = ldb;
  p.stage = static_cast<__nv_bfloat16*>(stage);
  p.slab_count = slab_count;
  p.world = world;
  p.rank = rank;
  p.wait_limit_ns = static_cast<unsigned long long>(wait_limit_ms > 0 ? wait_limit_ms : 2000) * 1000000ull;
  if (N % (256 * world) == 0) return launch_gather<256>(A, shards, stage, p, M, N, K, lda, ldb, world, rank, stream);
  return launch_gather<128>(A, shards, stage, p, M, N, K, lda, ldb, world, rank, stream);
}
