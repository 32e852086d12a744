"""Placeholder for the reference's sglang-jax engine (tunix/rl/rollout/sglang_jax_rollout.py:28-132).

sglang-jax is a JAX/TPU serving stack with no CUDA build; on this platform its role (paged KV
cache with `page_size`, chunked prefill, continuous batching, in-memory weight updates) is
filled by `NativeRollout`. Selecting `rollout_engine="sglang_jax"` therefore builds a
`NativeRollout` configured from the `rollout_sglang_jax_*` fields and says so once."""
from __future__ import annotations

import logging

from . import base_rollout, native_rollout


class SglangJaxRollout(native_rollout.NativeRollout):
  def __init__(self, model, tokenizer, rollout_config: base_rollout.RolloutConfig, mesh=None, **kwargs):
    logging.warning("rollout_engine='sglang_jax' has no CUDA implementation; using the native paged engine")
    page = getattr(rollout_config, "rollout_sglang_jax_page_size", None) or 16
    super().__init__(model, tokenizer, rollout_config, mesh=mesh, page_size=int(page))
