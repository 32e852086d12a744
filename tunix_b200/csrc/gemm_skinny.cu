// Skinny bf16 GEMM for decode steps (at most 128 activation rows against a large weight):
//
//   C[Mx, Nw] = epilogue( alpha * X[Mx, K] * W[Nw, K]^T )            Mx <= 128
//
// Such a product is bound by streaming W from HBM exactly once, so the kernel is organised
// around that stream rather than around output tiles:
//
//  * swapped operands: a 128-row slab of W is the M operand of tcgen05.mma (UMMA 128 x BNX x 16,
//    BNX = 16/32/64/128 >= Mx), the activations are the small N operand. Every byte of W that
//    arrives feeds a full-height MMA, whatever the batch size.
//  * split-K inside a thread-block cluster: decode weights have 32-200 slabs, fewer than the 148
//    SMs, so the K range of a slab is cut over the S CTAs of a cluster (S = 1..8 chosen per shape
//    so that slabs x S fills the machine). The partial accumulators never touch global memory:
//    each CTA owns 128/S of the slab's output columns, the others store their share of those
//    columns into a slot of the owner's shared memory (16-byte `st.shared::cluster` stores through
//    distributed shared memory), an mbarrier in the owner's shared memory counts the arrivals, and
//    the owner adds the S - 1 slots to its own accumulator in a fixed order and runs the epilogue.
//    One launch, no workspace, no atomics, no memset, no fix-up pass.
//  * deep TMA ring (3-12 stages of 16-32 KB of W), single-thread MMA issue, TMEM double-buffered
//    accumulators, four epilogue warps; clusters walk slabs persistently.
//
// Epilogues: bias, residual add (C = R + X W^T, C may alias R), and gated activations - with
// `glu` the weight is [gate rows | up rows] (2 x Nw rows), both slabs of a k-block are loaded and
// accumulated side by side in TMEM, and the epilogue writes act(gate) * up directly.
//
// Tensor-parallel exit (n_ranks > 1): every rank holds a K-shard of W, computes its partial
// product with the schedule above, stores each finished 128-column block of partial sums (fp32)
// into its own peer-mapped buffer and raises a per-block flag in every peer's flag table; the CTAs
// that finished a block then wait (bounded) for the same block of every peer, add the partials
// in rank order with plain peer loads over NVLink, and write the reduced bf16 result - the
// all-reduce overlaps the remaining slabs block by block, inside the GEMM kernel. No multicast
// object is involved. The call counter (`epoch`) lives in device memory and is advanced by the
// kernel itself, so a CUDA graph can replay the launch.
//
// With S = 1 (deterministic mode) a slab is reduced over K in one accumulator in k-block order, so
// repeated launches give identical bits. All TMA loads are plain (no cluster multicast).
#include "tx_host.h"
#include "tx_ptx.cuh"

namespace {

using namespace tx;

constexpr int BMW = 128;        // weight rows per slab (UMMA M)
constexpr int BK = 64;          // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int kMaxRanks = 8;
constexpr int kMaxFlagBlocks = 256;      // Nw <= 32768 on a tensor-parallel exit
constexpr int kMaxStages = 12;
constexpr int kMaxMyBlocks = 32;
constexpr int kSmemLimit = 227 * 1024;

struct SkinnyParams {
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* residual;   // optional [Mx, Nw], row stride ldr
  long long ldr;
  const __nv_bfloat16* bias;       // optional [Nw]
  int Mx, Nw, K;
  float alpha;
  int glu;                         // 0: none, 1: SiLU(gate) * up, 2: tanh-GELU(gate) * up
  int split;                       // S: CTAs per cluster = K ranges per slab
  int n_clusters;
  int stages;                      // TMA ring depth (fits beside the reduction buffers)
  int* status;
  // tensor-parallel exit
  int n_ranks, rank;
  float* part[kMaxRanks];          // rank r's partial buffer: [2 parities][part_stride] fp32
  int* flags[kMaxRanks];           // rank r's flag table: [n_ranks][kMaxFlagBlocks]
  long long part_stride;           // floats per parity
  int* epoch;                      // device call counter (same value on every rank)
  int* done;                       // CTAs of this launch that have finished
  unsigned long long wait_ns;
  // optional timeline: 16 globaltimer stamps per CTA (null = off); see tx_gemm_skinny_trace
  unsigned long long* trace;
};

template <int BNX, bool GLU>
struct SCfg {
  static constexpr int kAcc = GLU ? 2 : 1;
  static constexpr int kWBytes = BMW * BK * 2;
  static constexpr int kABytes = kWBytes * kAcc;
  static constexpr int kXBytes = BNX * BK * 2;
  static constexpr int kStageBytes = kABytes + kXBytes;
  static constexpr int kAccCols = kAcc * BNX;              // fp32 values per output column (TMEM lane)
  static constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;
};

// Exchange buffers of one CTA for a cluster of `split`: 2 parities x (split - 1) source slots x
// [rows_max][acc_cols + 4] floats (rows padded by 16 bytes so that a warp's 16-byte stores spread over the banks).
// A slab's 128 columns are owned in chunks of 8 (16 bytes of bf16 output): 16 chunks dealt out over the cluster.
__host__ __device__ inline int col_lo(int o, int split) { return 8 * ((16 * o + split - 1) / split); }
__host__ __device__ inline int rows_max_of(int split) { return 8 * ((16 + split - 1) / split); }
__host__ __device__ inline int slot_floats_of(int split, int acc_cols) { return rows_max_of(split) * (acc_cols + 4); }
__host__ __device__ inline int red_bytes_of(int split, int acc_cols) {
  return split > 1 ? 2 * (split - 1) * slot_floats_of(split, acc_cols) * 4 : 0;
}
// Columns [col_lo(o), col_lo(o + 1)) of a slab are finished by CTA `o` of the cluster.

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ void bar_epilogue() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier of the four epilogue warps that also tells whether `pred` held on every thread.
__device__ __forceinline__ bool bar_epilogue_all(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.u32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, 128, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t"
      "}\n"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred))
      : "memory");
  return r != 0;
}
// System-scope 16-byte read of a peer's partial sums.
__device__ __forceinline__ float4 ld_sys_f32x4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
// 16-byte store into the shared memory of another CTA of the cluster (address from map_to_cta).
__device__ __forceinline__ void st_dsmem_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait that makes the other CTAs' shared-memory writes visible (acquire at cluster scope).
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > TX_WAIT_LIMIT_NS) {
      *abort_flag = 1;
      return false;
    }
  }
}

// Records a phase boundary of this CTA when a trace buffer is attached.
__device__ __forceinline__ void stamp(const SkinnyParams& p, int slot) {
  if (p.trace) p.trace[blockIdx.x * 16 + slot] = globaltimer_ns();
}

// Final value of one output element from its accumulated product(s).
template <bool GLU>
__device__ __forceinline__ float activate(const SkinnyParams& p, float a, float u) {
  a *= p.alpha;
  if (GLU) {
    u *= p.alpha;
    a = (p.glu == 2 ? gelu_tanh_f(a) : silu_f(a)) * u;
  }
  return a;
}

template <int BNX, bool GLU>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                   const __grid_constant__ CUtensorMap map_x, const SkinnyParams p) {
  using C = SCfg<BNX, GLU>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int S = p.split, stages = p.stages;
  const int rows_max = rows_max_of(S);
  // layout: [stages x stage][reduction buffers, 2 parities][barriers and flags]
  float* redbuf = reinterpret_cast<float*>(smem_gen + stages * C::kStageBytes);
  const int red_bytes = red_bytes_of(S, C::kAccCols);
  // output staging: [BNX rows][128 columns] fp32, so that C is written in whole 16-byte pieces of a row
  float* stg = reinterpret_cast<float*>(smem_gen + stages * C::kStageBytes + red_bytes);
  constexpr int kStgBytes = BNX * BMW * 4;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + stages * C::kStageBytes + red_bytes + kStgBytes);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * kMaxStages;
  const uint32_t bar_tfull = bar_empty + 8 * kMaxStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  const uint32_t bar_red = bar_tempty + 16;       // [2]: contributions to my columns have arrived (per parity)
  const uint32_t bar_emit = bar_red + 16;         // tensor-parallel: every CTA of the cluster stored its part of a block
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kMaxStages + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* n_my_blocks = reinterpret_cast<volatile int*>(tmem_slot + 2);
  int* my_blocks = reinterpret_cast<int*>(tmem_slot + 3);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slabs = (p.Nw + BMW - 1) / BMW;
  const int num_kb = (p.K + BK - 1) / BK;
  const int crank = S > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int cluster_id = blockIdx.x / S;
  const int kb_lo = static_cast<int>(static_cast<long long>(num_kb) * crank / S);
  const int kb_hi = static_cast<int>(static_cast<long long>(num_kb) * (crank + 1) / S);
  const int my_lo = col_lo(crank, S), my_hi = col_lo(crank + 1, S);
  if (p.n_ranks > 1) griddep_wait();     // the call counter is written by the previous exit kernel of the chain
  const int epoch = p.n_ranks > 1 ? (*reinterpret_cast<volatile int*>(p.epoch) + 1) : 0;

  if (threadIdx.x == 0) {
    stamp(p, 0);                      // CTA started
    *abort_flag = 0;
    *n_my_blocks = 0;
    for (int s = 0; s < stages; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(bar_tfull + 8 * a, 1);
      mbar_init(bar_tempty + 8 * a, 128);
      mbar_init(bar_red + 8 * a, S > 1 ? (S - 1) * (my_hi - my_lo) : 1);
    }
    mbar_init(bar_emit, S);
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  if (S > 1) cluster_sync_all();      // everybody's barriers exist before anyone arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (threadIdx.x == 0) stamp(p, 1);    // set-up done (barriers, TMEM, cluster rendezvous)
  griddep_launch_dependents();          // a successor launched programmatically may take SMs as our CTAs leave

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&map_w);
      tma_prefetch_desc(&map_x);
      if (GLU) tma_prefetch_desc(&map_w2);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // The weights do not depend on the kernel before this one: the first pass over the ring issues its weight
      // tiles at once, then waits for the predecessor (programmatic dependent launch), then adds the activation
      // tiles to the same stages. From then on weight and activation tiles are issued together.
      const int per_slab = kb_hi - kb_lo;
      int early = 0;
      for (int slab = cluster_id; slab < slabs && early < stages; slab += p.n_clusters) {
        for (int kb = kb_lo; kb < kb_hi && early < stages; ++kb, ++early) {
          const uint32_t full = bar_full + 8 * early;
          const uint32_t sa = smem_base + early * C::kStageBytes;
          mbar_expect_tx(full, C::kStageBytes);
          tma_load_2d(sa, &map_w, kb * BK, slab * BMW, full);
          if (GLU) tma_load_2d(sa + C::kWBytes, &map_w2, kb * BK, slab * BMW, full);
          if (early == 0) stamp(p, 2);                                              // first load issued
        }
      }
      griddep_wait();
      {
        int q = 0;
        for (int slab = cluster_id; slab < slabs && q < early; slab += p.n_clusters)
          for (int kb = kb_lo; kb < kb_hi && q < early; ++kb, ++q)
            tma_load_2d(smem_base + q * C::kStageBytes + C::kABytes, &map_x, kb * BK, 0, bar_full + 8 * q);
      }
      stamp(p, 3);                                                                  // ring filled once
      stage = early % stages;
      phase = early == stages ? 1u : 0u;
      int q = 0;
      for (int slab = cluster_id; slab < slabs && ok; slab += p.n_clusters) {
        for (int kb = kb_lo; kb < kb_hi; ++kb, ++q) {
          if (q < early) continue;                                                  // issued above
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag)) {
            atomicOr(p.status, kStatusWaitTimeoutProducer);
            ok = false;
            break;
          }
          const uint32_t full = bar_full + 8 * stage;
          const uint32_t sa = smem_base + stage * C::kStageBytes;
          mbar_expect_tx(full, C::kStageBytes);
          tma_load_2d(sa, &map_w, kb * BK, slab * BMW, full);
          if (GLU) tma_load_2d(sa + C::kWBytes, &map_w2, kb * BK, slab * BMW, full);
          tma_load_2d(sa + C::kABytes, &map_x, kb * BK, 0, full);
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
      }
      (void)per_slab;
      stamp(p, 4);                                                                  // all loads issued
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BMW, BNX, false, false);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int slab = cluster_id; slab < slabs && ok; slab += p.n_clusters) {
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag)) {
          atomicOr(p.status, kStatusWaitTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * C::kAccCols;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
            atomicOr(p.status, kStatusWaitTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          if (slab == cluster_id && kb == kb_lo) stamp(p, 5);                       // first tile arrived
          const uint32_t sa = smem_base + stage * C::kStageBytes;
          const uint32_t sx = sa + C::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t dx = make_smem_desc_sw128(sx + k * 32, 16, 1024);
            const uint32_t accum = (kb > kb_lo || k > 0) ? 1u : 0u;
            umma_bf16(tmem_d, make_smem_desc_sw128(sa + k * 32, 16, 1024), dx, idesc, accum);
            if (GLU) umma_bf16(tmem_d + BNX, make_smem_desc_sw128(sa + C::kWBytes + k * 32, 16, 1024), dx, idesc, accum);
          }
          umma_commit(bar_empty + 8 * stage);
          if (++stage == stages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        umma_commit(bar_tfull + 8 * acc);
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        if (slab == cluster_id) stamp(p, 6);                                        // first slab: all MMAs issued
      }
      stamp(p, 7);                                                                  // last slab: all MMAs issued
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;              // TMEM lane quarter this warp may access
    const int col = quarter * 32 + lane;       // slab column (TMEM lane) of this thread
    const bool leader = (warp == 2 && lane == 0);
    const int owner = ((col >> 3) * S) >> 4;   // CTA of the cluster that finishes this column (8-column chunks)
    const bool mine = owner == crank;
    const int own_lo = col_lo(owner, S);
    float* part_self = p.n_ranks > 1 ? p.part[p.rank] + (epoch & 1) * p.part_stride : nullptr;
    griddep_wait();          // the residual (and C itself) belong to the kernels before this one
    int acc = 0, round = 0;
    uint32_t acc_phase = 0;
    for (int slab = cluster_id; slab < slabs; slab += p.n_clusters, ++round) {
      bool ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag);
      if (!ok) atomicOr(p.status, kStatusWaitTimeoutEpilogue);
      if (!bar_epilogue_all(ok)) break;          // all four warps leave together
      tc_fence_after();
      if (leader && round == 0) stamp(p, 8);     // first accumulator complete
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * C::kAccCols;
      const int par = round & 1;
      // tcgen05.ld is a warp-wide (.aligned) instruction: every branch that contains one is taken by whole warps.
      // A warp whose 32 columns belong to two owners (cluster sizes that do not divide 32 columns evenly) therefore
      // runs both phases, each lane acting only in the phase that matches its column.
      const bool warp_sends = !__all_sync(0xffffffffu, mine);
      const bool warp_finishes = __any_sync(0xffffffffu, mine);
      constexpr int kRow = C::kAccCols + 4;                       // floats per exchanged row
      const int slot_floats = rows_max * kRow;
      if (warp_sends) {
        // accumulator rows of columns that another CTA finishes: store them into my slot of that CTA's buffer
        const int my_slot = crank < owner ? crank : crank - 1;
        const uint32_t dst = map_to_cta(
            smem_u32(redbuf + (par * (S - 1) + my_slot) * slot_floats + (col - own_lo) * kRow), owner);
#pragma unroll 1
        for (int c = 0; c < C::kAccCols; c += 16) {
          if ((c & (BNX - 1)) >= p.Mx) continue;     // rows of X beyond Mx are zero-filled: nothing to send
          uint32_t r[16];
          tmem_ld_32x32b_x16(taddr + c, r);
          tmem_ld_wait();
          if (!mine) {
#pragma unroll
            for (int e = 0; e < 16; e += 4) st_dsmem_v4(dst + (c + e) * 4, r[e], r[e + 1], r[e + 2], r[e + 3]);
          }
        }
        if (!mine) mbar_arrive_cluster(map_to_cta(bar_red + 8 * par, owner));   // release: the stores are visible to the owner
      }
      if (warp_finishes) {
        if (S > 1) {
          // one lane polls (an acquire at cluster scope per poll is not cheap), the warp follows
          if (lane == 0 && !mbar_wait_cluster(bar_red + 8 * par, (round >> 1) & 1, abort_flag))
            atomicOr(p.status, kStatusWaitTimeoutEpilogue);
          __syncwarp();
          asm volatile("fence.acq_rel.cluster;" ::: "memory");
        }
        const float* mybuf = redbuf + par * (S - 1) * slot_floats + (col - own_lo) * kRow;
#pragma unroll 1
        for (int c = 0; c < BNX && c < p.Mx; c += 16) {
          uint32_t rg[16], ru[16];
          tmem_ld_32x32b_x16(taddr + c, rg);
          if (GLU) tmem_ld_32x32b_x16(taddr + BNX + c, ru);
          tmem_ld_wait();
          if (mine) {
            float a[16], u[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) { a[e] = __uint_as_float(rg[e]); u[e] = GLU ? __uint_as_float(ru[e]) : 0.f; }
            for (int sl = 0; sl < S - 1; ++sl) {               // slot order = rank order: a fixed summation order
              const float4* ga = reinterpret_cast<const float4*>(mybuf + sl * slot_floats + c);
              const float4* gu = reinterpret_cast<const float4*>(mybuf + sl * slot_floats + BNX + c);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float4 v = ga[q];
                a[4 * q] += v.x; a[4 * q + 1] += v.y; a[4 * q + 2] += v.z; a[4 * q + 3] += v.w;
                if (GLU) {
                  const float4 w = gu[q];
                  u[4 * q] += w.x; u[4 * q + 1] += w.y; u[4 * q + 2] += w.z; u[4 * q + 3] += w.w;
                }
              }
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) stg[(c + e) * BMW + col] = activate<GLU>(p, a[e], u[e]);
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      // ---- copy-out: all four warps move this CTA's columns of the staged tile, 8 outputs (16 bytes) at a time
      bar_epilogue();
      {
        const int nch = (my_hi - my_lo) >> 3;            // 8-column chunks this CTA finishes
        const int tid = (warp - 2) * 32 + lane;
        for (int idx = tid; idx < p.Mx * nch; idx += 128) {
          const int j = idx / nch, ch = idx - j * nch;
          const int cl = my_lo + ch * 8;                 // column within the slab
          const int n8 = slab * BMW + cl;
          if (n8 >= p.Nw) continue;                      // Nw is a multiple of 8: a chunk is inside or outside
          const float4 v0 = *reinterpret_cast<const float4*>(stg + j * BMW + cl);
          const float4 v1 = *reinterpret_cast<const float4*>(stg + j * BMW + cl + 4);
          float f[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
          if (p.n_ranks > 1) {
            float* dst = part_self + static_cast<long long>(j) * p.Nw + n8;
            *reinterpret_cast<float4*>(dst) = v0;
            *reinterpret_cast<float4*>(dst + 4) = v1;
            continue;
          }
          if (p.bias) {
            const uint4 b = *reinterpret_cast<const uint4*>(p.bias + n8);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
            for (int q = 0; q < 4; ++q) { const float2 t = __bfloat1622float2(b2[q]); f[2 * q] += t.x; f[2 * q + 1] += t.y; }
          }
          if (p.residual) {
            const uint4 r = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(j) * p.ldr + n8);
            const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
            for (int q = 0; q < 4; ++q) { const float2 t = __bfloat1622float2(r2[q]); f[2 * q] += t.x; f[2 * q + 1] += t.y; }
          }
          uint4 o;
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
          *reinterpret_cast<uint4*>(p.C + static_cast<long long>(j) * p.ldc + n8) = o;
        }
      }
      if (leader && round == 0) stamp(p, 9);     // first slab written

      if (p.n_ranks > 1) {
        // this CTA's columns of the block are in the rank's partial buffer; once all CTAs of the cluster say
        // so, its first CTA raises the block's flag on every rank. Everybody remembers the block for the reduction.
        __threadfence_system();
        bar_epilogue();
        if (leader) {
          if (S > 1) mbar_arrive_cluster(map_to_cta(bar_emit, 0));
          const int i = *n_my_blocks;
          if (i < kMaxMyBlocks) { my_blocks[i] = slab; *n_my_blocks = i + 1; }
          else atomicOr(p.status, kStatusBadArgument);
        }
        if (crank == 0 && warp == 2) {
          bool ready = true;
          if (S > 1) ready = mbar_wait_cluster(bar_emit, round & 1, abort_flag);
          __threadfence_system();
          if (ready && lane < p.n_ranks) st_release_sys(p.flags[lane] + p.rank * kMaxFlagBlocks + slab, epoch);
        }
      }
    }
    if (p.n_ranks > 1) {
      // ---------------------------------------------------------- all-reduce of the finished blocks
      bar_epilogue();
      const int nb = *n_my_blocks;
      const int* my_flags = p.flags[p.rank];
      for (int i = 0; i < nb; ++i) {
        const int blk = my_blocks[i];
        if (warp == 2 && lane < p.n_ranks) {
          const int* f = my_flags + lane * kMaxFlagBlocks + blk;
          const uint64_t t0 = globaltimer_ns();
          while (ld_acquire_sys(f) - epoch < 0) {
            if (*abort_flag) break;
            if (globaltimer_ns() - t0 > p.wait_ns) {
              atomicOr(p.status, kStatusPeerWaitTimeout);
              *abort_flag = 1;
              break;
            }
          }
        }
        if (!bar_epilogue_all(*abort_flag == 0)) break;
        // this CTA's columns of the block, 8 outputs at a time: sum the ranks' partials in rank order (every rank
        // computes the same bits), add bias and residual, round once
        const int nch = (my_hi - my_lo) >> 3;
        const int tid = (warp - 2) * 32 + lane;
        for (int idx = tid; idx < p.Mx * nch; idx += 128) {
          const int j = idx / nch, ch = idx - j * nch;
          const int n8 = blk * BMW + my_lo + ch * 8;
          if (n8 >= p.Nw) continue;
          const long long off = (epoch & 1) * p.part_stride + static_cast<long long>(j) * p.Nw + n8;
          float4 v[kMaxRanks][2];
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r) {
            if (r < p.n_ranks) {
              v[r][0] = ld_sys_f32x4(p.part[r] + off);
              v[r][1] = ld_sys_f32x4(p.part[r] + off + 4);
            }
          }
          float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r) {
            if (r < p.n_ranks) {
              f[0] += v[r][0].x; f[1] += v[r][0].y; f[2] += v[r][0].z; f[3] += v[r][0].w;
              f[4] += v[r][1].x; f[5] += v[r][1].y; f[6] += v[r][1].z; f[7] += v[r][1].w;
            }
          }
          if (p.bias) {
            const uint4 bb = *reinterpret_cast<const uint4*>(p.bias + n8);
            const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&bb);
#pragma unroll
            for (int q = 0; q < 4; ++q) { const float2 t = __bfloat1622float2(b2[q]); f[2 * q] += t.x; f[2 * q + 1] += t.y; }
          }
          if (p.residual) {
            const uint4 rr = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(j) * p.ldr + n8);
            const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&rr);
#pragma unroll
            for (int q = 0; q < 4; ++q) { const float2 t = __bfloat1622float2(r2[q]); f[2 * q] += t.x; f[2 * q + 1] += t.y; }
          }
          uint4 o;
          __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
          for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
          *reinterpret_cast<uint4*>(p.C + static_cast<long long>(j) * p.ldc + n8) = o;
        }
      }
    }
  }

  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) stamp(p, 10);   // all roles done
  // No rendezvous at exit: peers store into this CTA's shared memory only before they arrive on its exchange
  // barrier, and this CTA has waited for every such arrival before it got here.
  if (threadIdx.x == 0) { stamp(p, 11); if (p.trace) { p.trace[blockIdx.x * 16 + 12] = S; p.trace[blockIdx.x * 16 + 13] = stages; } }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (p.n_ranks > 1 && threadIdx.x == 0) {
    // the last CTA to leave advances the call counter for the next launch (or graph replay)
    __threadfence();
    const int old = atomicAdd(p.done, 1);
    if (old == static_cast<int>(gridDim.x) - 1) {
      *p.done = 0;
      *p.epoch = epoch;
      __threadfence();
    }
  }
}

// 1: launch with programmatic stream serialization, so that set-up and the first weight tiles overlap the tail of
// the kernel before (which must have been launched on the same stream). Off: an ordinary launch.
static int g_pdl = [] {
  const char* e = getenv("TUNIX_B200_PDL");
  return (e && e[0] == '0') ? 0 : 1;
}();

// Per (kernel, device, split) cache of how many clusters can be resident at once.
struct ClusterFit {
  int stages[9] = {};
  int max_clusters[9] = {};
  bool known[9] = {};
};

template <int BNX, bool GLU>
int launch_skinny(const void* X, const void* W, SkinnyParams p, long long ldx, long long ldw, int deterministic,
                  int max_ctas, cudaStream_t stream) {
  using C = SCfg<BNX, GLU>;
  auto kern = gemm_skinny_kernel<BNX, GLU>;
  static txh::DeviceFlag attr_flag;
  static ClusterFit fits[txh::kMaxDevices];
  bool& attr_set = attr_flag.cur();
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit) != cudaSuccess) return 300;
    attr_set = true;
  }
  ClusterFit& fit = fits[txh::current_device()];
  const int slabs = (p.Nw + BMW - 1) / BMW, num_kb = (p.K + BK - 1) / BK;
  int sms = txh::sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;

  constexpr int kStg = BNX * BMW * 4;       // output staging tile
  auto smem_for = [&](int split, int stages) { return stages * C::kStageBytes + red_bytes_of(split, C::kAccCols) + kStg + 1024 + 512; };
  auto probe = [&](int split) {
    if (fit.known[split]) return;
    fit.known[split] = true;
    int stages = (kSmemLimit - red_bytes_of(split, C::kAccCols) - kStg - 1024 - 512) / C::kStageBytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 3) return;                          // not worth it: max_clusters stays 0
    fit.stages[split] = stages;
    if (split == 1) { fit.max_clusters[1] = txh::sm_count(); return; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(split * txh::sm_count(), 1, 1);
    cfg.blockDim = dim3(NUM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem_for(split, stages);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) { (void)cudaGetLastError(); n = 0; }
    fit.max_clusters[split] = n;
  };

  // Pick the split whose schedule streams the weight in the fewest k-block steps: rounds x k-blocks per CTA,
  // plus a charge per round for pipeline start-up and, when K is split, the exchange of partial sums (measured:
  // about 1.3 us resp. 3.4 us, i.e. 4 resp. 10 k-block times).
  int best_s = 1, best_nc = 1;
  long long best_cost = -1;
  const int max_split = deterministic ? 1 : 8;
  for (int s = 1; s <= max_split; ++s) {
    if (s > 1 && num_kb / s < 4) break;              // every CTA keeps at least 4 k-blocks
    probe(s);
    int nc = fit.max_clusters[s];
    if (nc > sms / s) nc = sms / s;
    if (nc < 1) continue;
    if (nc > slabs) nc = slabs;
    const int rounds = (slabs + nc - 1) / nc;
    const long long cost = static_cast<long long>(rounds) * ((num_kb + s - 1) / s + (s > 1 ? 10 : 4));
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best_s = s; best_nc = nc; }
  }
  if (best_cost < 0) return 301;
  static const bool verbose = [] { const char* e = getenv("TUNIX_B200_SKINNY_VERBOSE"); return e && e[0] == '1'; }();
  if (verbose) {
    fprintf(stderr, "[gemm_skinny] rows<=%d glu=%d N=%d K=%d slabs=%d kblocks=%d -> split %d x %d clusters; resident clusters by split:",
            BNX, GLU ? 1 : 0, p.Nw, p.K, slabs, num_kb, best_s, best_nc);
    for (int s = 1; s <= 8; ++s) fprintf(stderr, " %d:%d", s, fit.known[s] ? fit.max_clusters[s] : -1);
    fprintf(stderr, "\n");
  }
  p.split = best_s;
  p.n_clusters = best_nc;
  p.stages = fit.stages[best_s];
  if (p.n_ranks > 1 && (slabs + best_nc - 1) / best_nc > kMaxMyBlocks) return 4;

  CUtensorMap mw, mw2, mx;
  int rc = txh::make_map_2d_bf16(&mw, W, p.Nw, p.K, ldw, BMW, BK);
  if (rc) return 100 + rc;
  mw2 = mw;
  if (GLU) {
    rc = txh::make_map_2d_bf16(&mw2, static_cast<const __nv_bfloat16*>(W) + static_cast<long long>(p.Nw) * ldw, p.Nw,
                               p.K, ldw, BMW, BK);
    if (rc) return 100 + rc;
  }
  rc = txh::make_map_2d_bf16(&mx, X, p.Mx, p.K, ldx, BNX, BK);
  if (rc) return 200 + rc;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(best_nc * best_s, 1, 1);
  cfg.blockDim = dim3(NUM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem_for(best_s, p.stages);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = best_s;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl ? 2 : 1;
  if (cudaLaunchKernelEx(&cfg, kern, mw, mw2, mx, p) != cudaSuccess) { (void)cudaGetLastError(); return 400; }
  return 0;
}

template <bool GLU>
int dispatch_bnx(int Mx, const void* X, const void* W, const SkinnyParams& p, long long ldx, long long ldw,
                 int deterministic, int max_ctas, cudaStream_t stream) {
  if (Mx <= 16) return launch_skinny<16, GLU>(X, W, p, ldx, ldw, deterministic, max_ctas, stream);
  if (Mx <= 32) return launch_skinny<32, GLU>(X, W, p, ldx, ldw, deterministic, max_ctas, stream);
  if (Mx <= 64) return launch_skinny<64, GLU>(X, W, p, ldx, ldw, deterministic, max_ctas, stream);
  return launch_skinny<128, GLU>(X, W, p, ldx, ldw, deterministic, max_ctas, stream);
}

}  // namespace

extern "C" int tx_gemm_skinny_flag_blocks() { return kMaxFlagBlocks; }
extern "C" int tx_gemm_skinny_set_pdl(int on) {
  const int before = g_pdl;
  g_pdl = on ? 1 : 0;
  return before;
}

// Debug aid: attaches (or, with null, detaches) a device buffer of 16 x 64-bit words per CTA (room for 8 * SM count
// CTAs) that later launches fill with %globaltimer stamps of their phase boundaries: 0 start, 1 set-up done, 2 first
// load issued, 3 ring filled, 4 all loads issued, 5 first tile arrived, 6 / 7 MMAs of the first / last slab issued,
// 8 first accumulator complete, 9 first slab written, 10 roles done, 11 exit; 12 cluster size, 13 ring depth.
static unsigned long long* g_trace = nullptr;
extern "C" void tx_gemm_skinny_trace(unsigned long long* buf) { g_trace = buf; }

// C[Mx, Nw] = epilogue(alpha * X W^T); see the top of this file.
//   X [Mx, K] bf16 (row stride ldx), W [Nw, K] bf16 - with glu != 0, [2 Nw, K]: gate rows then up rows - (row
//   stride ldw), C [Mx, Nw] bf16 (row stride ldc). Bases 16-byte aligned, ldx / ldw multiples of 8, Mx <= 128.
//   deterministic != 0: a slab is never split over CTAs, so repeated launches give identical bits.
//   max_ctas > 0 caps the number of CTAs.
// Tensor-parallel exit when n_ranks > 1 (no glu): part[r] / flags[r] are rank r's peer-mapped partial buffer
// (2 * part_stride floats, part_stride >= Mx * Nw) and flag table (n_ranks * tx_gemm_skinny_flag_blocks() ints,
// zero-initialised); epoch / done are two zero-initialised device ints private to this rank. Every rank of the
// group must issue the same sequence of calls, and the kernel must be able to have all its CTAs resident.
extern "C" int tx_gemm_skinny(const void* X, const void* W, void* C, const void* residual, const void* bias, int Mx,
                              int Nw, int K, long long ldx, long long ldw, long long ldc, long long ldr, float alpha,
                              int glu, int deterministic, int* status, int max_ctas, int n_ranks, int rank,
                              void* const* part, void* const* flags, long long part_stride, int* epoch, int* done,
                              long long wait_ms, cudaStream_t stream) {
  if (Mx <= 0 || Mx > 128 || Nw <= 0 || K <= 0 || glu < 0 || glu > 2) return 1;
  if ((ldx & 7) || (ldw & 7) || (ldc & 7) || (Nw & 7) || (residual && (ldr & 7)) || !status) return 2;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15) ||
      (reinterpret_cast<uintptr_t>(C) & 15) || (reinterpret_cast<uintptr_t>(residual) & 15) ||
      (reinterpret_cast<uintptr_t>(bias) & 15))
    return 3;
  if (glu && ((static_cast<long long>(Nw) * ldw * 2) & 15)) return 3;
  if (n_ranks > 1) {
    if (glu || n_ranks > kMaxRanks || rank < 0 || rank >= n_ranks || !part || !flags || !epoch || !done) return 4;
    if ((Nw + BMW - 1) / BMW > kMaxFlagBlocks || part_stride < static_cast<long long>(Mx) * Nw) return 4;
  }
  SkinnyParams p{};
  p.C = static_cast<__nv_bfloat16*>(C);
  p.ldc = ldc;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldr = ldr;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.Mx = Mx; p.Nw = Nw; p.K = K;
  p.alpha = alpha;
  p.glu = glu;
  p.status = status;
  p.trace = g_trace;
  p.n_ranks = n_ranks > 1 ? n_ranks : 1;
  p.rank = rank;
  if (n_ranks > 1) {
    for (int r = 0; r < n_ranks; ++r) {
      if (!part[r] || !flags[r]) return 4;
      p.part[r] = static_cast<float*>(part[r]);
      p.flags[r] = static_cast<int*>(flags[r]);
    }
    p.part_stride = part_stride;
    p.epoch = epoch;
    p.done = done;
    p.wait_ns = static_cast<unsigned long long>(wait_ms > 0 ? wait_ms : 2000) * 1000000ull;
  }
  return glu ? dispatch_bnx<true>(Mx, X, W, p, ldx, ldw, deterministic, max_ctas, stream)
             : dispatch_bnx<false>(Mx, X, W, p, ldx, ldw, deterministic, max_ctas, stream);
}
