"""Rollout throughput of the paged engine on random-init weights.

  python -m benchmarks.rollout_bench --model qwen3_8b --prompts 64 --samples 8 --prompt-len 256 --new-tokens 768

Prints one JSON line: generated tokens/s (device-timed with CUDA events around the whole
`generate`, prefill included), decode steps and their mean latency.
"""
from __future__ import annotations

import argparse
import json

import numpy as np
import torch

from tunix_b200.models import automodel, dummy_model_creator
from tunix_b200.models.transformer import Transformer
from tunix_b200.rollout import EngineConfig, PagedEngine


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--model", default="qwen3_8b")
  ap.add_argument("--layers", type=int, default=0)
  ap.add_argument("--prompts", type=int, default=64)
  ap.add_argument("--samples", type=int, default=8)
  ap.add_argument("--prompt-len", type=int, default=256)
  ap.add_argument("--new-tokens", type=int, default=768)
  ap.add_argument("--max-batch", type=int, default=512)
  ap.add_argument("--no-graphs", action="store_true")
  ap.add_argument("--warmup-tokens", type=int, default=8)
  ap.add_argument("--page-size", type=int, default=16)
  a = ap.parse_args()
  cfg = automodel.call_model_config(a.model)
  if a.layers:
    import dataclasses
    cfg = dataclasses.replace(cfg, num_layers=a.layers)
  model = dummy_model_creator.create_dummy_model(Transformer, cfg, dtype=torch.bfloat16, device="cuda").eval()
  eng = PagedEngine(model, EngineConfig(page_size=a.page_size, max_batch=a.max_batch, max_seq_len=a.prompt_len + a.new_tokens + 16,
                                        use_cuda_graphs=not a.no_graphs))
  rng = np.random.default_rng(0)
  prompts = [rng.integers(0, cfg.vocab_size, size=a.prompt_len).tolist() for _ in range(a.prompts)]
  prompts = [p for p in prompts for _ in range(a.samples)]
  eng.generate(prompts, a.warmup_tokens, temperature=1.0, seed=1)          # captures the graphs
  torch.cuda.synchronize()
  s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  s.record()
  res = eng.generate(prompts, a.new_tokens, temperature=1.0, seed=2)
  e.record()
  torch.cuda.synchronize()
  ms = s.elapsed_time(e)
  n = sum(len(t) for t in res.tokens)
  print(json.dumps({"metric": "rollout generated tokens/s", "value": round(n / ms * 1e3, 1), "ms": round(ms, 1),
                    "generated": n, "decode_steps": res.steps, "ms_per_decode_step": round(ms / max(res.steps, 1), 3),
                    "prefill_ms": round(res.prefill_ms, 1),
                    "decode_only_ms_per_step": round((ms - res.prefill_ms) / max(res.steps, 1), 3),
                    "sequences": len(prompts), "model": a.model, "layers": cfg.num_layers,
                    "cuda_graphs": not a.no_graphs, "page_size": a.page_size, "kv_cache_gb": round(eng.cache.bytes() / 2 ** 30, 1),
                    "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1)}))


if __name__ == "__main__":
  main()
