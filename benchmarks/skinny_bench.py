"""Decode-shaped (skinny) GEMM micro-benchmark: the stream-K kernel (`tx_gemm_skinny`) against the
general tcgen05 GEMM of this package and `torch.nn.functional.linear` (library), Qwen3-8B shapes.

    python -m benchmarks.skinny_bench [--rows 16 64 128] [--iters 30] [--graph]

Each timed launch follows a 256 MB write (cold L2) and is timed with CUDA events; the median is
reported in microseconds with the weight-streaming rate (weight bytes / time) as a fraction of
`--copy-gbs` (the measured device copy bandwidth). `--graph` times 36 back-to-back launches of
each shape inside one CUDA graph instead (warm pipeline, no launch gaps: what a decode step sees).
"""
from __future__ import annotations

import argparse
import json

import torch

from tunix_b200.ops import _lib, kernels

SHAPES = [("qkv", 6144, 4096), ("o_proj", 4096, 4096), ("gate_up+glu", 24576, 4096), ("down", 4096, 12288),
          ("lm_head", 151936, 4096)]


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--rows", type=int, nargs="+", default=[16, 64, 128])
  ap.add_argument("--iters", type=int, default=30)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--copy-gbs", type=float, default=6549.4)
  ap.add_argument("--graph", action="store_true")
  ap.add_argument("--only", default="")
  ap.add_argument("--trace", action="store_true",
                  help="print the kernel's own phase timeline (median over CTAs, microseconds since the first CTA start)")
  a = ap.parse_args(argv)
  flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

  def timeit(fn):
    for _ in range(a.warmup):
      fn()
    torch.cuda.synchronize()
    if a.graph:
      g = torch.cuda.CUDAGraph()
      with torch.cuda.graph(g):
        for _ in range(36):
          fn()
      g.replay()
      torch.cuda.synchronize()
      ts = []
      for _ in range(5):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / 36)
      ts.sort()
      return ts[len(ts) // 2]
    ts = []
    for _ in range(a.iters):
      flush.zero_()
      e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      e0.record()
      fn()
      e1.record()
      torch.cuda.synchronize()
      ts.append(e0.elapsed_time(e1) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]

  for M in a.rows:
    for name, N, K in SHAPES:
      if a.only and a.only not in name:
        continue
      glu = name.startswith("gate_up")
      x = (torch.randn(M, K, device="cuda") * 0.5).to(torch.bfloat16)
      # in graph mode 36 distinct weights defeat L2 reuse between the launches of one replay
      nw = 36 if a.graph and N * K * 2 < (300 << 20) else 1
      ws = [(torch.randn(N, K, device="cuda") * 0.05).to(torch.bfloat16) for _ in range(nw)]
      state = {"i": 0}

      def w():
        state["i"] = (state["i"] + 1) % nw
        return ws[state["i"]]

      wbytes = N * K * 2
      row = {"rows": M, "shape": name, "N": N, "K": K, "weight_mb": round(wbytes / 2 ** 20, 1)}
      t = timeit(lambda: kernels.gemm_skinny(x, w(), glu="silu" if glu else None))
      row["skinny_us"] = round(t, 1)
      if a.trace:
        import ctypes
        lib = _lib.require()
        lib.tx_gemm_skinny_trace.argtypes = [ctypes.c_void_p]
        lib.tx_gemm_skinny_trace.restype = None
        buf = torch.zeros(8 * 160 * 16, dtype=torch.int64, device="cuda")
        flush.zero_()
        lib.tx_gemm_skinny_trace(buf.data_ptr())
        kernels.gemm_skinny(x, w(), glu="silu" if glu else None)
        torch.cuda.synchronize()
        lib.tx_gemm_skinny_trace(None)
        tr = buf.view(-1, 16).cpu()
        tr = tr[tr[:, 0] > 0]
        t0 = int(tr[:, 0].min())
        names = ["start", "setup_done", "first_load", "ring_filled", "loads_issued", "first_tile", "mma_first_slab",
                 "mma_last_slab", "acc_ready", "slab_written", "roles_done", "exit"]
        med = {n: round(float((tr[:, i][tr[:, i] > 0] - t0).float().median()) / 1e3, 2) for i, n in enumerate(names)
               if (tr[:, i] > 0).any()}
        mx = {n: round(float((tr[:, i][tr[:, i] > 0] - t0).float().max()) / 1e3, 2) for i, n in enumerate(names)
              if (tr[:, i] > 0).any()}
        row["trace"] = {"ctas": int(tr.shape[0]), "cluster": int(tr[0, 12]), "stages": int(tr[0, 13]), "median_us": med,
                        "max_us": mx}
      row["skinny_frac_of_copy"] = round(wbytes / (t * 1e-6) / 1e9 / a.copy_gbs, 3)
      if M % 8 == 0:
        if glu:
          t = timeit(lambda: kernels.glu_fwd(kernels.gemm(x, w()), False))
        else:
          t = timeit(lambda: kernels.gemm(x, w()))
        row["general_us"] = round(t, 1)
      if glu:
        def lib_fn():
          gu = torch.nn.functional.linear(x, w())
          return torch.nn.functional.silu(gu[:, :N // 2]) * gu[:, N // 2:]
        t = timeit(lib_fn)
      else:
        t = timeit(lambda: torch.nn.functional.linear(x, w()))
      row["library_us"] = round(t, 1)
      row["library_frac_of_copy"] = round(wbytes / (t * 1e-6) / 1e9 / a.copy_gbs, 3)
      _lib.check_status()
      print(json.dumps(row), flush=True)
      del ws


if __name__ == "__main__":
  main()
