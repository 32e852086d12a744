"""TFLOP accounting (tunix/sft/system_metrics_calculator.py:23-76).

The reference reads XLA's cost analysis; here FLOPs come from the model configuration
(`tunix_b200.models.flops.train_flops_per_token`) or, lacking one, from the 6 * params
heuristic.
"""
from __future__ import annotations

import logging
from typing import Any, Optional

log = logging.getLogger(__name__)


def measure_tflops_per_step(model: Any, tokens_per_step: int, seq_len: Optional[int] = None) -> Optional[float]:
  """TFLOPs of one training step (forward + backward) from the model's config; None if unknown."""
  cfg = getattr(model, "config", None)
  try:
    from tunix_b200.models import flops
    if cfg is not None:
      return flops.train_flops_per_token(cfg, seq_len or 1) * tokens_per_step / 1e12
  except Exception as e:  # pragma: no cover
    log.debug("flops from config failed: %s", e)
  n = sum(p.numel() for p in model.parameters()) if hasattr(model, "parameters") else None
  return None if n is None else 6.0 * n * tokens_per_step / 1e12


def approximate_tflops_per_second(total_model_params: int, global_batch_size: int, step_time_delta: float) -> float:
  """`6 * B * params / dt` in TFLOP/s. Inputs that cannot give a rate (no parameters, no batch, no elapsed time: the
  first step of a run, a clock that did not advance) give 0.0 and a warning rather than ending the training loop
  over a metric."""
  if total_model_params <= 0 or global_batch_size <= 0 or step_time_delta <= 0:
    log.warning("TFLOPS cannot be approximated from params=%s, batch size=%s, step time=%s: all must be positive.",
                total_model_params, global_batch_size, step_time_delta)
    return 0.0
  return 6.0 * global_batch_size * total_model_params / step_time_delta / 1e12
