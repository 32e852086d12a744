"""Times the grouped expert GEMM (`csrc/gemm_grouped.cu`) on mixture-of-experts shapes.

    python -m benchmarks.moe_bench                       # Qwen3-30B-A3B: E 128, top-8, D 2048, F 768
    python -m benchmarks.moe_bench --tokens 2048 --iters 3 --warmup 1     # small case for a profiler

Prints one JSON line per product (forward, dgrad, wgrad of gate|up and of down) with CUDA-event times,
useful TFLOP/s (padding rows not counted) and, for comparison, the per-expert loop of dense GEMMs.
"""
from __future__ import annotations

import argparse
import json

import torch

from tunix_b200.ops import kernels
from tunix_b200.ops import moe as moe_ops


def _time(fn, iters, warmup, flush):
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  ms = []
  for _ in range(iters):
    flush.add_(1.0)                      # a 256 MB write pushes the previous iteration's operands out of L2
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    ms.append(e0.elapsed_time(e1))
  ms.sort()
  return ms[len(ms) // 2]


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--tokens", type=int, default=8192)
  ap.add_argument("--experts", type=int, default=128)
  ap.add_argument("--top-k", type=int, default=8)
  ap.add_argument("--dim", type=int, default=2048)
  ap.add_argument("--ffn", type=int, default=768)
  ap.add_argument("--iters", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--no-loop", action="store_true", help="skip the per-expert loop comparison")
  a = ap.parse_args()
  dev = torch.device("cuda")
  torch.manual_seed(0)
  E, k, D, Fh, T = a.experts, a.top_k, a.dim, a.ffn, a.tokens
  n = T * k
  ids = torch.stack([torch.randperm(E, device=dev)[:k] for _ in range(T)]).reshape(-1)
  lay = moe_ops.padded_layout(ids, E)
  flush = torch.zeros(64 * 2**20, dtype=torch.float32, device=dev)
  bf = torch.bfloat16
  for name, N, K in (("gate_up", 2 * Fh, D), ("down", D, Fh)):
    w = torch.randn(E, N, K, device=dev, dtype=bf) * 0.02
    x = torch.zeros(lay.rows, K, device=dev, dtype=bf)
    x[lay.dest] = torch.randn(n, K, device=dev, dtype=bf)
    dy = torch.zeros(lay.rows, N, device=dev, dtype=bf)
    dy[lay.dest] = torch.randn(n, N, device=dev, dtype=bf)
    y = torch.zeros(lay.rows, N, device=dev, dtype=bf)
    dx = torch.zeros(lay.rows, K, device=dev, dtype=bf)
    dw = torch.zeros(E, N, K, device=dev, dtype=torch.float32)
    fl = 2.0 * n * N * K
    runs = {
        "fwd": lambda: moe_ops._call(0, x, w, y, lay, N, K, E),
        "dgrad": lambda: moe_ops._call(1, dy, w, dx, lay, N, K, E),
        "wgrad_fp32_acc": lambda: moe_ops._call(2, dy, x, dw, lay, N, K, E, accumulate=True),
    }
    for kind, fn in runs.items():
      ms = _time(fn, a.iters, a.warmup, flush)
      print(json.dumps({"kernel": "gemm_grouped", "proj": name, "product": kind, "rows": n, "padded_rows": lay.rows,
                        "E": E, "N": N, "K": K, "ms": round(ms, 4), "useful_tflops": round(fl / ms / 1e9, 1)}))
    if not a.no_loop:
      off = lay.offsets.tolist()
      def loop():
        for e in range(E):
          if off[e + 1] > off[e]:
            kernels.gemm(x[off[e]:off[e + 1]], w[e], out=y[off[e]:off[e + 1]])
      ms = _time(loop, max(2, a.iters // 4), 1, flush)
      print(json.dumps({"kernel": "per-expert loop of dense GEMMs", "proj": name, "product": "fwd", "ms": round(ms, 4),
                        "useful_tflops": round(fl / ms / 1e9, 1)}))


if __name__ == "__main__":
  main()
