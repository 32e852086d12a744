"""GEMM micro-benchmark: the tcgen05 kernels of this package against torch.matmul (cuBLAS).

    python -m benchmarks.gemm_bench                       # Llama-8B training shapes
    python -m benchmarks.gemm_bench --shape 8192 6144 4096 --iters 3 --no-cublas

Every timed call is preceded by a write larger than L2, timed with CUDA events; the median is
reported in TFLOP/s. Layouts: tn = forward (x W^T), nn = dgrad, nt = wgrad.
"""
from __future__ import annotations

import argparse
import json

import torch

from tunix_b200.ops import _lib, kernels

DEFAULT_SHAPES = [(8192, 6144, 4096), (8192, 4096, 4096), (8192, 28672, 4096), (8192, 4096, 14336),
                  (4096, 6144, 4096), (4096, 28672, 4096), (4096, 4096, 14336), (2048, 128256, 4096)]


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--shape", type=int, nargs=3, action="append", metavar=("M", "N", "K"))
  ap.add_argument("--iters", type=int, default=10)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--no-cublas", action="store_true")
  ap.add_argument("--single-cta", action="store_true", help="force the 1-CTA kernels")
  a = ap.parse_args(argv)
  shapes = [tuple(s) for s in a.shape] if a.shape else DEFAULT_SHAPES
  flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
  if a.single_cta:
    _lib.require().tx_gemm_set_disable_pair(1)

  def timeit(fn):
    for _ in range(a.warmup):
      fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(a.iters):
      flush.zero_()
      e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      e0.record()
      fn()
      e1.record()
      torch.cuda.synchronize()
      ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]

  for M, N, K in shapes:
    x = torch.randn(M, K, device="cuda").to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    xt, wt = x.t().contiguous(), w.t().contiguous()
    fl = 2.0 * M * N * K
    row = {"M": M, "N": N, "K": K}
    row["tx_tn"] = fl / timeit(lambda: kernels.gemm(x, w)) / 1e9
    row["tx_nn"] = fl / timeit(lambda: kernels.gemm(x, wt, b_mn=True)) / 1e9
    row["tx_nt"] = fl / timeit(lambda: kernels.gemm(xt, wt, a_mn=True, b_mn=True)) / 1e9
    acc = torch.zeros(M, N, device="cuda", dtype=torch.float32)
    row["tx_nt_acc_f32"] = fl / timeit(lambda: kernels.gemm(xt, wt, a_mn=True, b_mn=True, out=acc, accumulate=True)) / 1e9
    if not a.no_cublas:
      row["cublas_nt_acc_f32"] = fl / timeit(lambda: acc.add_(torch.matmul(xt.t(), wt))) / 1e9
      row["cublas_tn"] = fl / timeit(lambda: torch.matmul(x, w.t())) / 1e9
      row["cublas_nt"] = fl / timeit(lambda: torch.matmul(xt.t(), wt)) / 1e9
    _lib.check_status()
    print(json.dumps({k: (round(v, 1) if isinstance(v, float) else v) for k, v in row.items()}), flush=True)


if __name__ == "__main__":
  main()
