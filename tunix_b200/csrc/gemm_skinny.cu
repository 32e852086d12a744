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
//  * stream-K: the (weight slab, k-block) space is cut into one contiguous range per CTA, one CTA
//    per SM, so all SMs pull the same number of bytes. A slab whose k-blocks are shared by several
//    CTAs is summed in an fp32 scratch slot with `red.global.add`; the CTA that completes the slab
//    (a counter tells it) applies the epilogue, writes C and leaves slot and counter zeroed, so the
//    product is ONE launch - no memset before and no conversion pass after.
//  * deep TMA ring (4-12 stages of 16-32 KB of W), single-thread MMA issue, TMEM double-buffered
//    accumulators, four epilogue warps.
//
// Epilogues: bias, residual add (C = R + X W^T, C may alias R), and gated activations - with
// `glu` the weight is [gate rows | up rows] (2 x Nw rows), both slabs of a k-block are loaded and
// accumulated side by side in TMEM, and the epilogue writes act(gate) * up directly.
//
// Tensor-parallel exit (n_ranks > 1): every rank holds a K-shard of W, computes its partial
// product with the schedule above, stores each finished 128-column block of partial sums (fp32)
// into its own peer-mapped buffer and raises a per-block flag in every peer's flag table; the CTA
// that finished a block then waits (bounded) for the same block of every peer, adds the partials
// in rank order with plain peer loads over NVLink, and writes the reduced bf16 result - the
// all-reduce overlaps the remaining slabs block by block, inside the GEMM kernel. No multicast
// object is involved. The call counter (`epoch`) lives in device memory and is advanced by the
// kernel itself, so a CUDA graph can replay the launch.
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
constexpr int kSlotFloats = 2 * 128 * 128;   // scratch slot: [gate|up][BNX <= 128 rows][128 columns]

struct SkinnyParams {
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* residual;   // optional [Mx, Nw], row stride ldr
  long long ldr;
  const __nv_bfloat16* bias;       // optional [Nw]
  int Mx, Nw, K;
  float alpha;
  int glu;                         // 0: none, 1: SiLU(gate) * up, 2: tanh-GELU(gate) * up
  int whole_slabs;                 // 1: no slab is shared between CTAs (bitwise reproducible)
  float* ws;                       // gridDim.x slots of kSlotFloats floats, zero between launches
  int* counters;                   // gridDim.x ints, zero between launches
  int* status;
  // tensor-parallel exit
  int n_ranks, rank;
  float* part[kMaxRanks];          // rank r's partial buffer: [2 parities][part_rows * part_ld] fp32
  int* flags[kMaxRanks];           // rank r's flag table: [n_ranks][kMaxFlagBlocks]
  long long part_stride;           // floats per parity
  int* epoch;                      // device call counter (same value on every rank)
  int* done;                       // CTAs of this launch that have finished
  unsigned long long wait_ns;
};

template <int BNX, bool GLU>
struct SCfg {
  static constexpr int kAcc = GLU ? 2 : 1;
  static constexpr int kWBytes = BMW * BK * 2;
  static constexpr int kABytes = kWBytes * kAcc;
  static constexpr int kXBytes = BNX * BK * 2;
  static constexpr int kStageBytes = kABytes + kXBytes;
  static constexpr int kFit = (227 * 1024 - 4096) / kStageBytes;
  static constexpr int kStages = kFit > 12 ? 12 : kFit;
  static constexpr int kAccCols = kAcc * BNX;
  static constexpr int kTmemCols = 2 * kAccCols < 32 ? 32 : 2 * kAccCols;
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 512 /*barriers, flags*/;
};

// The k-block ranges (slab, [k0, k1)) of one CTA, in order.
class Segments {
 public:
  __device__ Segments(int slabs, int kb, int ctas, int cta, bool whole) : slabs_(slabs), kb_(kb), ctas_(ctas), whole_(whole) {
    if (whole) {
      slab_ = cta;
    } else {
      const long long total = static_cast<long long>(slabs) * kb;
      pos_ = total * cta / ctas;
      end_ = total * (cta + 1) / ctas;
    }
  }
  __device__ bool next(int& slab, int& k0, int& k1) {
    if (whole_) {
      if (slab_ >= slabs_) return false;
      slab = slab_; k0 = 0; k1 = kb_;
      slab_ += ctas_;
      return true;
    }
    if (pos_ >= end_) return false;
    slab = static_cast<int>(pos_ / kb_);
    const long long base = static_cast<long long>(slab) * kb_;
    const long long stop = end_ < base + kb_ ? end_ : base + kb_;
    k0 = static_cast<int>(pos_ - base);
    k1 = static_cast<int>(stop - base);
    pos_ = stop;
    return true;
  }

 private:
  int slabs_, kb_, ctas_;
  bool whole_;
  int slab_ = 0;
  long long pos_ = 0, end_ = 0;
};

// Scratch slot of a shared slab: the CTA whose range holds the slab's first k-block. Two shared
// slabs never map to one CTA (a CTA's range cannot contain the first block of two slabs without
// containing the whole of the earlier one).
__device__ __forceinline__ int slot_of(int slab, int kb, int slabs, int ctas) {
  const long long total = static_cast<long long>(slabs) * kb, x = static_cast<long long>(slab) * kb;
  int g = static_cast<int>(x * ctas / total);
  while (g + 1 < ctas && total * (g + 1) / ctas <= x) ++g;
  while (g > 0 && total * g / ctas > x) --g;
  return g;
}

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
// L2 reads of data other CTAs produced with reductions (never cached in L1).
__device__ __forceinline__ float4 ld_cg_f32x4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
// System-scope reads of a peer's buffer.
__device__ __forceinline__ float4 ld_sys_f32x4(const float* p) {
  float4 v;
  asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
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

// Writes one finished value: into this rank's partial buffer on a tensor-parallel exit, else to C.
__device__ __forceinline__ void emit(const SkinnyParams& p, float* part_self, int j, int n, float v) {
  if (p.n_ranks > 1) {
    part_self[static_cast<long long>(j) * p.Nw + n] = v;
    return;
  }
  if (p.bias) v += __bfloat162float(p.bias[n]);
  if (p.residual) v += __bfloat162float(p.residual[static_cast<long long>(j) * p.ldr + n]);
  p.C[static_cast<long long>(j) * p.ldc + n] = __float2bfloat16_rn(v);
}

// Four finished values of row j, columns n .. n + 3 (n a multiple of 4, n + 3 < Nw).
__device__ __forceinline__ void emit4(const SkinnyParams& p, float* part_self, int j, int n, float4 v) {
  if (p.n_ranks > 1) {
    *reinterpret_cast<float4*>(part_self + static_cast<long long>(j) * p.Nw + n) = v;
    return;
  }
  if (p.bias) {
    const uint2 b = *reinterpret_cast<const uint2*>(p.bias + n);
    const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
    const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
    v.x += b0.x; v.y += b0.y; v.z += b1.x; v.w += b1.y;
  }
  if (p.residual) {
    const uint2 r = *reinterpret_cast<const uint2*>(p.residual + static_cast<long long>(j) * p.ldr + n);
    const float2 r0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
    const float2 r1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
    v.x += r0.x; v.y += r0.y; v.z += r1.x; v.w += r1.y;
  }
  uint2 o;
  *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p.C + static_cast<long long>(j) * p.ldc + n) = o;
}

template <int BNX, bool GLU>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_w2,
                   const __grid_constant__ CUtensorMap map_x, const SkinnyParams p) {
  using C = SCfg<BNX, GLU>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_gen + C::kStages * C::kStageBytes);
  const uint32_t bar_full = smem_u32(bars);
  const uint32_t bar_empty = bar_full + 8 * C::kStages;
  const uint32_t bar_tfull = bar_empty + 8 * C::kStages;
  const uint32_t bar_tempty = bar_tfull + 16;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * C::kStages + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_slot + 2);
  int* my_blocks = reinterpret_cast<int*>(tmem_slot + 4);      // blocks this CTA has to reduce (<= 24)
  volatile int* n_my_blocks = reinterpret_cast<volatile int*>(tmem_slot + 3);
  constexpr int kMaxMyBlocks = 24;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int slabs = (p.Nw + BMW - 1) / BMW;
  const int num_kb = (p.K + BK - 1) / BK;
  const int ctas = gridDim.x, cta = blockIdx.x;
  const bool whole = p.whole_slabs != 0;
  const int epoch = p.n_ranks > 1 ? (*reinterpret_cast<volatile int*>(p.epoch) + 1) : 0;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *last_flag = 0;
    *n_my_blocks = 0;
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
      tma_prefetch_desc(&map_w);
      tma_prefetch_desc(&map_x);
      if (GLU) tma_prefetch_desc(&map_w2);
      Segments seg(slabs, num_kb, ctas, cta, whole);
      int slab, k0, k1, stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (ok && seg.next(slab, k0, k1)) {
        for (int kb = k0; kb < k1; ++kb) {
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
          if (++stage == C::kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BMW, BNX, false, false);
      Segments seg(slabs, num_kb, ctas, cta, whole);
      int slab, k0, k1, stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      while (ok && seg.next(slab, k0, k1)) {
        if (!mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag)) {
          atomicOr(p.status, kStatusWaitTimeoutMma);
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + acc * C::kAccCols;
        for (int kb = k0; kb < k1; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, abort_flag)) {
            atomicOr(p.status, kStatusWaitTimeoutMma);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * C::kStageBytes;
          const uint32_t sx = sa + C::kABytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t dx = make_smem_desc_sw128(sx + k * 32, 16, 1024);
            const uint32_t accum = (kb > k0 || k > 0) ? 1u : 0u;
            umma_bf16(tmem_d, make_smem_desc_sw128(sa + k * 32, 16, 1024), dx, idesc, accum);
            if (GLU) umma_bf16(tmem_d + BNX, make_smem_desc_sw128(sa + C::kWBytes + k * 32, 16, 1024), dx, idesc, accum);
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
    const int quarter = warp & 3;              // TMEM lane quarter this warp may access
    const int col = quarter * 32 + lane;       // column of the slab this thread owns
    const bool leader = (warp == 2 && lane == 0);
    float* part_self = p.n_ranks > 1 ? p.part[p.rank] + (epoch & 1) * p.part_stride : nullptr;
    Segments seg(slabs, num_kb, ctas, cta, whole);
    int slab, k0, k1, acc = 0;
    uint32_t acc_phase = 0;
    while (seg.next(slab, k0, k1)) {
      bool ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag);
      if (!ok) atomicOr(p.status, kStatusWaitTimeoutEpilogue);
      if (!bar_epilogue_all(ok)) break;          // all four warps leave together
      tc_fence_after();
      const int n = slab * BMW + col;
      const bool complete = (k0 == 0 && k1 == num_kb);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * C::kAccCols;
      float* slot = nullptr;
      int slot_idx = 0;
      if (!complete) {
        slot_idx = slot_of(slab, num_kb, slabs, ctas);
        slot = p.ws + static_cast<long long>(slot_idx) * kSlotFloats;
      }
#pragma unroll 1
      for (int c = 0; c < BNX; c += 16) {
        uint32_t rg[16], ru[16];
        tmem_ld_32x32b_x16(taddr + c, rg);
        if (GLU) tmem_ld_32x32b_x16(taddr + BNX + c, ru);
        tmem_ld_wait();
        if (complete) {
          if (n < p.Nw) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const int j = c + e;
              if (j < p.Mx)
                emit(p, part_self, j, n, activate<GLU>(p, __uint_as_float(rg[e]), GLU ? __uint_as_float(ru[e]) : 0.f));
            }
          }
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const int j = c + e;
            if (j < p.Mx) {
              atomicAdd(slot + j * BMW + col, __uint_as_float(rg[e]));
              if (GLU) atomicAdd(slot + (BNX + j) * BMW + col, __uint_as_float(ru[e]));
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(bar_tempty + 8 * acc);
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }

      bool finished_block = complete;
      if (!complete) {
        // publish this CTA's share; whoever brings the slab's k-block count to num_kb finishes it
        __threadfence();
        bar_epilogue();
        if (leader) {
          __threadfence();
          const int old = atomicAdd(p.counters + slot_idx, k1 - k0);
          *last_flag = (old + (k1 - k0) == num_kb) ? 1 : 0;
          if (*last_flag) __threadfence();
        }
        bar_epilogue();
        if (*last_flag) {
          finished_block = true;
          // thread -> 4 columns x every 4th row; 8 rows of loads in flight at a time
          const int c4 = (col & 31) * 4, r0 = col >> 5;
          const int n4 = slab * BMW + c4;
          for (int jb = r0; jb < p.Mx; jb += 32) {
            float4 a[8], u[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int j = jb + 4 * e;
              if (j < p.Mx) {
                a[e] = ld_cg_f32x4(slot + j * BMW + c4);
                if (GLU) u[e] = ld_cg_f32x4(slot + (BNX + j) * BMW + c4);
              }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int j = jb + 4 * e;
              if (j < p.Mx) {
                *reinterpret_cast<float4*>(slot + j * BMW + c4) = make_float4(0.f, 0.f, 0.f, 0.f);
                if (GLU) *reinterpret_cast<float4*>(slot + (BNX + j) * BMW + c4) = make_float4(0.f, 0.f, 0.f, 0.f);
                if (n4 < p.Nw) {
                  float4 v;
                  v.x = activate<GLU>(p, a[e].x, GLU ? u[e].x : 0.f);
                  v.y = activate<GLU>(p, a[e].y, GLU ? u[e].y : 0.f);
                  v.z = activate<GLU>(p, a[e].z, GLU ? u[e].z : 0.f);
                  v.w = activate<GLU>(p, a[e].w, GLU ? u[e].w : 0.f);
                  emit4(p, part_self, j, n4, v);
                }
              }
            }
          }
          if (leader) p.counters[slot_idx] = 0;
        }
        bar_epilogue();       // last_flag is rewritten by the next shared slab
      }
      if (finished_block && p.n_ranks > 1) {
        // the block of partial sums is in this rank's buffer: tell every rank, remember to reduce it
        __threadfence_system();
        bar_epilogue();
        if (lane < p.n_ranks && warp == 2)
          st_release_sys(p.flags[lane] + p.rank * kMaxFlagBlocks + slab, epoch);
        if (leader) {
          const int i = *n_my_blocks;
          if (i < kMaxMyBlocks) { my_blocks[i] = slab; *n_my_blocks = i + 1; }
          else atomicOr(p.status, kStatusBadArgument);
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
        const int c4 = (col & 31) * 4, r0 = col >> 5;
        const int n4 = blk * BMW + c4;
        if (n4 < p.Nw) {
          const long long off = (epoch & 1) * p.part_stride + n4;
          float4 bias = make_float4(0.f, 0.f, 0.f, 0.f);
          if (p.bias) {
            const uint2 b = *reinterpret_cast<const uint2*>(p.bias + n4);
            const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.x));
            const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b.y));
            bias = make_float4(b0.x, b0.y, b1.x, b1.y);
          }
          for (int jb = r0; jb < p.Mx; jb += 16) {
            float4 v[4][kMaxRanks];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j = jb + 4 * e;
#pragma unroll
              for (int r = 0; r < kMaxRanks; ++r)
                if (r < p.n_ranks && j < p.Mx) v[e][r] = ld_sys_f32x4(p.part[r] + off + static_cast<long long>(j) * p.Nw);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int j = jb + 4 * e;
              if (j >= p.Mx) continue;
              float4 s = bias;
#pragma unroll
              for (int r = 0; r < kMaxRanks; ++r)       // rank order: every rank computes the same bits
                if (r < p.n_ranks) { s.x += v[e][r].x; s.y += v[e][r].y; s.z += v[e][r].z; s.w += v[e][r].w; }
              if (p.residual) {
                const uint2 q = *reinterpret_cast<const uint2*>(p.residual + static_cast<long long>(j) * p.ldr + n4);
                const float2 q0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.x));
                const float2 q1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&q.y));
                s.x += q0.x; s.y += q0.y; s.z += q1.x; s.w += q1.y;
              }
              uint2 o;
              *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(s.x, s.y);
              *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(s.z, s.w);
              *reinterpret_cast<uint2*>(p.C + static_cast<long long>(j) * p.ldc + n4) = o;
            }
          }
        }
      }
    }
  }

  if (*abort_flag) __nanosleep(200000);
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
  if (p.n_ranks > 1 && threadIdx.x == 0) {
    // the last CTA to leave advances the call counter for the next launch (or graph replay)
    __threadfence();
    const int old = atomicAdd(p.done, 1);
    if (old == ctas - 1) {
      *p.done = 0;
      *p.epoch = epoch;
      __threadfence();
    }
  }
}

template <int BNX, bool GLU>
int launch_skinny(const void* X, const void* W, const SkinnyParams& p, long long ldx, long long ldw, int grid,
                  cudaStream_t stream) {
  using C = SCfg<BNX, GLU>;
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
  auto kern = gemm_skinny_kernel<BNX, GLU>;
  static txh::DeviceFlag attr_flag;
  bool& attr_set = attr_flag.cur();
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes) != cudaSuccess) return 300;
    attr_set = true;
  }
  kern<<<grid, NUM_THREADS, C::kSmemBytes, stream>>>(mw, mw2, mx, p);
  return cudaGetLastError() == cudaSuccess ? 0 : 400;
}

template <bool GLU>
int dispatch_bnx(int Mx, const void* X, const void* W, const SkinnyParams& p, long long ldx, long long ldw, int grid,
                 cudaStream_t stream) {
  if (Mx <= 16) return launch_skinny<16, GLU>(X, W, p, ldx, ldw, grid, stream);
  if (Mx <= 32) return launch_skinny<32, GLU>(X, W, p, ldx, ldw, grid, stream);
  if (Mx <= 64) return launch_skinny<64, GLU>(X, W, p, ldx, ldw, grid, stream);
  return launch_skinny<128, GLU>(X, W, p, ldx, ldw, grid, stream);
}

}  // namespace

// Number of scratch slots (= the largest grid) and floats per slot that `tx_gemm_skinny` may use.
extern "C" int tx_gemm_skinny_slots() { return txh::sm_count(); }
extern "C" int tx_gemm_skinny_slot_floats() { return kSlotFloats; }
extern "C" int tx_gemm_skinny_flag_blocks() { return kMaxFlagBlocks; }

// C[Mx, Nw] = epilogue(alpha * X W^T); see the top of this file.
//   X [Mx, K] bf16 (row stride ldx), W [Nw, K] bf16 - with glu != 0, [2 Nw, K]: gate rows then up rows - (row
//   stride ldw), C [Mx, Nw] bf16 (row stride ldc). Bases 16-byte aligned, ldx / ldw multiples of 8, Mx <= 128.
//   ws: tx_gemm_skinny_slots() * tx_gemm_skinny_slot_floats() floats, counters: tx_gemm_skinny_slots() ints; both
//   zero before the first call and left zero by every call; launches sharing them must be ordered on one stream.
//   deterministic != 0: no slab is shared between CTAs, so repeated launches give identical bits.
//   max_ctas > 0 caps the grid.
// Tensor-parallel exit when n_ranks > 1 (no glu): part[r] / flags[r] are rank r's peer-mapped partial buffer
// (2 * part_stride floats, part_stride >= Mx * Nw) and flag table (n_ranks * tx_gemm_skinny_flag_blocks() ints,
// zero-initialised); epoch / done are two zero-initialised device ints private to this rank. Every rank of the
// group must issue the same sequence of calls, and the kernel must be able to have all its CTAs resident.
extern "C" int tx_gemm_skinny(const void* X, const void* W, void* C, const void* residual, const void* bias, int Mx,
                              int Nw, int K, long long ldx, long long ldw, long long ldc, long long ldr, float alpha,
                              int glu, int deterministic, float* ws, int* counters, int* status, int max_ctas,
                              int n_ranks, int rank, void* const* part, void* const* flags, long long part_stride,
                              int* epoch, int* done, long long wait_ms, cudaStream_t stream) {
  if (Mx <= 0 || Mx > 128 || Nw <= 0 || K <= 0 || glu < 0 || glu > 2) return 1;
  if ((ldx & 7) || (ldw & 7) || (ldc & 7) || (Nw & 7) || (residual && (ldr & 7)) || !ws || !counters || !status) return 2;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) return 3;
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
  p.ws = ws;
  p.counters = counters;
  p.status = status;
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
  const int slabs = (Nw + BMW - 1) / BMW, num_kb = (K + BK - 1) / BK;
  int sms = txh::sm_count();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  int grid;
  if (deterministic) {
    p.whole_slabs = 1;
    grid = slabs < sms ? slabs : sms;
  } else {
    // every CTA gets at least 4 k-blocks; with fewer the fix-up costs more than the balance gains
    const long long total = static_cast<long long>(slabs) * num_kb;
    long long g = total / 4;
    if (g < 1) g = 1;
    grid = static_cast<int>(g < sms ? g : sms);
    // a tensor-parallel CTA remembers at most 24 finished blocks
    p.whole_slabs = 0;
  }
  if (n_ranks > 1 && (slabs + grid - 1) / grid + 2 > 24) return 4;
  return glu ? dispatch_bnx<true>(Mx, X, W, p, ldx, ldw, grid, stream)
             : dispatch_bnx<false>(Mx, X, W, p, ldx, ldw, grid, stream);
}
