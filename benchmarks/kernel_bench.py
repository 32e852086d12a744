"""Times the memory-bound kernels one at a time and prints achieved bandwidth.

  python -m benchmarks.kernel_bench [--only rmsnorm_fwd,paged_decode] [--iters 10]

Every case works on more bytes than the L2 holds, is warmed up, and is timed
with CUDA events around `iters` back-to-back launches. "bytes" is the
algorithmic traffic (each input read once, each output written once). One JSON
line per kernel: name, shape, ms, GB/s, and the fraction of the measured copy
bandwidth when a peaks file is found beside the package.
"""

from __future__ import annotations

import argparse
import json
import os

import torch

from tunix_b200.ops import kernels as K
from tunix_b200.ops import paged


def _time(fn, iters, warmup=3):
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  a.record()
  for _ in range(iters):
    fn()
  b.record()
  torch.cuda.synchronize()
  return a.elapsed_time(b) / iters


def _peak_gbs():
  here = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
  try:
    with open(os.path.join(here, "MEASURED_PEAKS.json")) as f:
      return float(json.load(f)["hbm_gbs"]), "measured"
  except (OSError, KeyError, ValueError):
    return 6650.0, "fallback"


def cases(dev, small=False):
  bf = torch.bfloat16
  T, D, F, V = (4096 if small else 16384), 4096, 14336, 128256
  out = {}

  def rms_fwd():
    x = torch.randn(T, D, device=dev, dtype=bf); r = torch.randn_like(x)
    w = torch.ones(D, device=dev, dtype=bf)
    return (lambda: K.rmsnorm_fwd(x, w, 1e-6, 0.0, r), 4 * T * D * 2, f"T={T} D={D} +residual")
  out["rmsnorm_fwd"] = rms_fwd

  def rms_bwd():
    x = torch.randn(T, D, device=dev, dtype=bf); dy = torch.randn_like(x); dres = torch.randn_like(x)
    w = torch.ones(D, device=dev, dtype=bf)
    _, _, rstd = K.rmsnorm_fwd(x, w, 1e-6)
    return (lambda: K.rmsnorm_bwd(x, w, dy, rstd, 1e-6, 0.0, dres), 4 * T * D * 2, f"T={T} D={D} +dres")
  out["rmsnorm_bwd"] = rms_bwd

  def glu_f():
    gu = torch.randn(T, 2 * F, device=dev, dtype=bf)
    return (lambda: K.glu_fwd(gu, False), 3 * T * F * 2, f"T={T} F={F} silu")
  out["glu_fwd"] = glu_f

  def glu_b():
    gu = torch.randn(T, 2 * F, device=dev, dtype=bf); do = torch.randn(T, F, device=dev, dtype=bf)
    return (lambda: K.glu_bwd(gu, do, False), 5 * T * F * 2, f"T={T} F={F} silu")
  out["glu_bwd"] = glu_b

  def lp_f():
    t = 1024 if small else 4096
    lg = torch.randn(t, V, device=dev, dtype=bf); tg = torch.randint(0, V, (t,), device=dev)
    return (lambda: K.logprob_fwd(lg, tg), t * V * 2, f"T={t} V={V} bf16 logits")
  out["logprob_fwd"] = lp_f

  def lp_b():
    t = 1024 if small else 4096
    lg = torch.randn(t, V, device=dev, dtype=bf); tg = torch.randint(0, V, (t,), device=dev)
    logp, lse, _ = K.logprob_fwd(lg, tg)
    g = torch.ones(t, device=dev); o = torch.empty_like(lg)
    return (lambda: K.logprob_bwd(lg, tg, lse, None, g, None, out=o), 2 * t * V * 2, f"T={t} V={V}")
  out["logprob_bwd"] = lp_b

  def adamw():
    n = (64 if small else 256) << 20
    master = torch.randn(n, device=dev); m = torch.zeros(n, device=dev); v = torch.zeros(n, device=dev)
    g = torch.randn(n, device=dev); p = torch.empty(n, device=dev, dtype=bf)
    return (lambda: K.adamw_step(master, m, v, g, p, lr=1e-4, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                                 step=3), n * (4 * 4 * 2 + 2), f"n={n} fp32 grad, zeroed in place")
  out["adamw"] = adamw

  def make_decode(page, L=640):
    def decode():
      B, N, Kh, H = (128 if small else 512), 32, 8, 128
      blocks = (L + page - 1) // page
      P = B * blocks
      kp = torch.randn(P, page, Kh, H, device=dev, dtype=bf); vp = torch.randn_like(kp)
      bt = torch.randperm(P, device=dev, dtype=torch.int32).view(B, blocks).contiguous()
      lens = torch.full((B,), L, device=dev, dtype=torch.int32)
      q = torch.randn(B, N, H, device=dev, dtype=bf)
      return (lambda: paged.paged_decode_attention(q, kp, vp, bt, lens, H ** -0.5, max_len=L),
              2 * B * L * Kh * H * 2 + 2 * B * N * H * 2, f"B={B} N={N} Kh={Kh} H={H} len={L} page={page}")
    return decode
  out["paged_decode"] = make_decode(16)
  out["paged_decode_p64"] = make_decode(64)
  out["paged_decode_p64_len1000"] = make_decode(64, 1000)

  def sample():
    B, Vq = 512, 151936
    lg = torch.randn(B, Vq, device=dev, dtype=bf)
    return (lambda: paged.sample(lg, 1.0, False, seed=1, step=2), B * Vq * 2, f"B={B} V={Vq} bf16")
  out["sample"] = sample

  def allgather_gemm():
    # the all-gather-into-GEMM kernel with 4 "ranks" whose shards all live on this GPU (one launch)
    from tunix_b200.ops import kernels
    M, N, K, world = (2048 if small else 8192), 8192, 4096, 4
    x = torch.randn(M, K, device=dev, dtype=bf)
    shards = [torch.randn(N // world, K, device=dev, dtype=bf) * 0.02 for _ in range(world)]
    stage = torch.empty(N, K, device=dev, dtype=bf)
    cnt = torch.empty(N // 128, device=dev, dtype=torch.int32)
    c = torch.empty(M, N, device=dev, dtype=bf)
    ptrs = [t.data_ptr() for t in shards]
    return (lambda: kernels.gemm_allgather_b(x, ptrs, 1, N // world, stage, cnt, out=c),
            (M * K + N * K + M * N) * 2 + (world - 1) * (N // world) * K * 2 * 2,
            f"M={M} N={N} K={K} world={world} (2*M*N*K = {2 * M * N * K / 1e12:.2f} TFLOP)")
  out["allgather_gemm"] = allgather_gemm

  def moe_rows():
    # single-rank dispatch -> combine of routed rows (the kernels the expert-parallel path runs over peer memory)
    from tunix_b200.ops import moe as moe_ops
    T, k, D, E = (2048 if small else 8192), 8, 2048, 128
    x = torch.randn(T, D, device=dev, dtype=bf)
    ids = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).reshape(-1)
    lay = moe_ops.padded_layout(ids, E)
    dest = lay.dest.int()
    zero = torch.zeros_like(dest)
    w = torch.rand(T * k, device=dev)

    def run():
      buf = moe_ops._dispatch_rows(x, k, None, dest, zero, lay.rows)
      moe_ops._combine_rows(buf, w, k, T, dest, zero, keep_rows=False)
    return (run, (lay.rows * D + T * D + 2 * T * k * D + T * D) * 2, f"T={T} k={k} D={D} E={E} rows={lay.rows}")
  out["moe_dispatch_combine"] = moe_rows
  return out


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--only", default="")
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--small", action="store_true", help="about a quarter of the bytes (for profiler captures)")
  a = ap.parse_args()
  dev = torch.device("cuda", 0)
  peak, how = _peak_gbs()
  table = cases(dev, a.small)
  names = [n for n in a.only.split(",") if n] or list(table)
  for name in names:
    fn, nbytes, shape = table[name]()
    ms = _time(fn, a.iters, a.warmup)
    gbs = nbytes / ms / 1e6
    print(json.dumps({"kernel": name, "shape": shape, "ms": round(ms, 4), "GB_s": round(gbs, 1),
                      f"frac_of_{how}_copy": round(gbs / peak, 3)}), flush=True)
    del fn
    torch.cuda.empty_cache()


if __name__ == "__main__":
  main()
