"""Times the tcgen05 flash attention forward against the library flash kernel.

  python -m benchmarks.flash_bench --batch 2 --seq 4096 --heads 32 --kv-heads 8 [--iters 20] [--no-lib]

Prints one JSON line per implementation: ms per call and TFLOP/s (causal FLOPs = 2 * B*N*L*L*H).
"""
from __future__ import annotations

import argparse
import json
import math

import torch

from tunix_b200.ops import _lib, flash


def _time(fn, iters, warmup):
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  s.record()
  for _ in range(iters):
    fn()
  e.record()
  torch.cuda.synchronize()
  return s.elapsed_time(e) / iters


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--batch", type=int, default=2)
  ap.add_argument("--seq", type=int, default=4096)
  ap.add_argument("--heads", type=int, default=32)
  ap.add_argument("--kv-heads", type=int, default=8)
  ap.add_argument("--iters", type=int, default=20)
  ap.add_argument("--warmup", type=int, default=3)
  ap.add_argument("--full", action="store_true", help="non-causal")
  ap.add_argument("--no-lib", action="store_true")
  a = ap.parse_args()
  B, L, N, K, H = a.batch, a.seq, a.heads, a.kv_heads, 128
  causal = not a.full
  qkv = torch.randn(B, L, (N + 2 * K) * H, device="cuda").bfloat16()
  q = qkv[..., :N * H].view(B, L, N, H)
  k = qkv[..., N * H:(N + K) * H].view(B, L, K, H)
  v = qkv[..., (N + K) * H:].view(B, L, K, H)
  scale = 1 / math.sqrt(H)
  flops = 4.0 * B * N * L * L * H * (0.5 if causal else 1.0)
  ms = _time(lambda: flash.forward(q, k, v, causal=causal, scale=scale), a.iters, a.warmup)
  _lib.check_status()
  print(json.dumps({"impl": "tx_flash_fwd", "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1),
                    "shape": [B, L, N, K, H], "causal": causal}))
  o, ctx = flash.forward(q, k, v, causal=causal, scale=scale)
  do = torch.randn_like(o)
  dqkv = torch.empty_like(qkv)
  dq, dk, dv = (dqkv[..., :N * H].view(B, L, N, H), dqkv[..., N * H:(N + K) * H].view(B, L, K, H),
                dqkv[..., (N + K) * H:].view(B, L, K, H))
  ms = _time(lambda: flash.backward(do, q, k, v, o, ctx, dq, dk, dv), a.iters, a.warmup)
  _lib.check_status()
  print(json.dumps({"impl": "tx_flash_bwd", "ms": round(ms, 4), "tflops": round(2.5 * flops / ms / 1e9, 1)}))
  if not a.no_lib:
    e = torch.empty(0, dtype=torch.long, device="cuda")
    ot, dot, lse = o.transpose(1, 2), do.transpose(1, 2), ctx[1]
    fnb = lambda: torch.ops.aten._scaled_dot_product_flash_attention_backward(
        dot, q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), ot, lse, None, None, L, L, 0.0, causal, e, e,
        scale=scale)
    ms = _time(fnb, a.iters, a.warmup)
    print(json.dumps({"impl": "library_flash_bwd", "ms": round(ms, 4), "tflops": round(2.5 * flops / ms / 1e9, 1)}))
  if not a.no_lib:
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    fn = lambda: torch.ops.aten._scaled_dot_product_flash_attention(qt, kt, vt, 0.0, causal, False, scale=scale)
    ms = _time(fn, a.iters, a.warmup)
    print(json.dumps({"impl": "library_flash", "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1)}))


if __name__ == "__main__":
  main()
