"""`rollout_engine="sglang_jax"` (tunix/rl/rollout/sglang_jax_rollout.py:28-132).

sglang-jax is a JAX/TPU serving stack with no CUDA build. What it contributes to a rollout - a paged KV cache with
a configurable page size, chunked prefill, a cap on running requests, padded batch buckets compiled ahead of time,
in-memory weight updates - is what the native paged engine does on this platform, so the engine name is kept and
its `rollout_sglang_jax_*` configuration is *translated* (`engine_geometry`) instead of ignored:

  page_size                     -> KV page size, clamped to what the paged-attention kernels take (8..64 tokens)
  context_length                -> per-sequence KV budget (never below prompt + generation)
  max_running_requests          -> sequences decoded together
  chunked_prefill_size          -> tokens per prefill forward (-1 / None: engine default)
  precompile_bs_paddings        -> recorded as `geometry["warm_buckets"]` (decode graphs are captured on first use of
                                   a bucket, which costs milliseconds here, not a compilation)
  mem_fraction_static           -> cap on the KV pool, as a fraction of the GPU's memory
  enable_deterministic_sampling -> fixed reduction order in the decode GEMMs for the lifetime of the engine

Knobs that only make sense for the JAX engine (`load_format`, `use_sort_for_toppk_minp`, single-process mode, static
LoRA slots) are accepted and reported once as having no effect.
"""
from __future__ import annotations

import logging
from typing import Any, Dict, List, Optional

import torch

from . import base_rollout, native_rollout

_MIN_PAGE, _MAX_PAGE = 8, 64
_NO_EFFECT = ("rollout_sglang_jax_load_format", "rollout_sglang_jax_use_sort_for_toppk_minp",
              "rollout_sglang_jax_enable_single_process", "rollout_sglang_jax_enable_static_lora",
              "rollout_sglang_jax_model_version", "rollout_sglang_jax_disable_radix_cache")


def _bytes_per_token(model_config: Any, dtype_bytes: int = 2) -> int:
  return 2 * model_config.num_layers * model_config.num_kv_heads * model_config.head_dim * dtype_bytes


def engine_geometry(rc: base_rollout.RolloutConfig, model_config: Any, device_memory_bytes: Optional[int] = None
                    ) -> Dict[str, Any]:
  """The paged engine's geometry implied by the sglang-jax fields of a rollout config."""
  get = lambda name, default=None: getattr(rc, f"rollout_sglang_jax_{name}", default)
  page = int(get("page_size") or 16)
  page = max(_MIN_PAGE, min(_MAX_PAGE, 1 << (page.bit_length() - 1)))            # power of two inside the kernel range
  need = rc.max_prompt_length + rc.max_tokens_to_generate
  max_seq = max(need, int(get("context_length") or 0), int(getattr(rc, "kv_cache_size", 0) or 0))
  max_batch = int(get("max_running_requests") or native_rollout.DEFAULT_MAX_BATCH)
  geometry: Dict[str, Any] = {"page_size": page, "max_seq_len": max_seq, "max_batch": max_batch}
  chunk = get("chunked_prefill_size")
  if chunk is not None and int(chunk) > 0:
    geometry["max_prefill_tokens"] = max(page, int(chunk))
  buckets = get("precompile_bs_paddings")
  if buckets:
    geometry["warm_buckets"] = sorted({min(int(b), max_batch) for b in buckets if int(b) > 0})
  fraction = float(get("mem_fraction_static") or 0.0)
  if device_memory_bytes and 0.0 < fraction <= 1.0:
    per_page = page * _bytes_per_token(model_config)
    wanted = max_batch * -(-max_seq // page)
    geometry["num_pages"] = max(max_batch, min(wanted, int(fraction * device_memory_bytes) // per_page))
  return geometry


class SglangJaxRollout(native_rollout.NativeRollout):

  def __init__(self, model, tokenizer, rollout_config: base_rollout.RolloutConfig, mesh=None, **kwargs):
    set_knobs = [k for k in _NO_EFFECT if getattr(rollout_config, k, None) not in (None, "", "auto", True, False)]
    logging.warning("rollout_engine='sglang_jax' runs on the native paged engine on this platform%s",
                    f"; no effect here: {set_knobs}" if set_knobs else "")
    device = next(model.parameters()).device
    memory = torch.cuda.get_device_properties(device).total_memory if device.type == "cuda" else None
    self.geometry = engine_geometry(rollout_config, model.config, memory)
    super().__init__(model, tokenizer, rollout_config, mesh=mesh, page_size=self.geometry["page_size"],
                     max_batch=self.geometry["max_batch"], engine_overrides=self.geometry)
    self._fixed_order = None
    if getattr(rollout_config, "rollout_sglang_jax_enable_deterministic_sampling", False):
      from ...ops import kernels
      self._fixed_order = kernels.fixed_reduction_order()
      self._fixed_order.__enter__()

  def close(self) -> None:
    if self._fixed_order is not None:
      self._fixed_order.__exit__(None, None, None)
      self._fixed_order = None
    closer = getattr(super(), "close", None)
    if callable(closer):
      closer()
