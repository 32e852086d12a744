"""Trainer utilities: masks, positions, weighted metrics and loss outputs.

Semantics follow tunix/sft/utils.py:33-232: positions are 0-based from the first valid
token, the causal mask is `mask[:, None, :] & tril`, and `WeightedMetric` defers the division
so that gradient accumulation yields the global weighted mean instead of a mean of means.
"""
from __future__ import annotations

import contextlib
import dataclasses
import gc
import logging
import time
from typing import Any, Mapping, Optional, Union

import torch

log = logging.getLogger(__name__)


def make_causal_attn_mask(input_mask: torch.Tensor) -> torch.Tensor:
  """[B, L] validity mask -> [B, L, L] boolean attention mask (True = may attend)."""
  if input_mask.dim() != 2:
    raise ValueError(f"Input mask must be 2D (shape [B, L]), but got {tuple(input_mask.shape)}.")
  L = input_mask.shape[-1]
  causal = torch.ones(L, L, dtype=torch.bool, device=input_mask.device).tril()
  return input_mask.bool()[:, None, :] & causal[None]


def build_positions_from_mask(input_mask: torch.Tensor) -> torch.Tensor:
  """cumsum(mask) - 1 clipped at 0: indices for RoPE given a padding mask."""
  pos = torch.cumsum(input_mask.long(), dim=-1)
  return pos - (pos >= 1).long()


def is_lora_enabled(model: torch.nn.Module) -> bool:
  """True if any parameter of the model is a LoRA adapter parameter."""
  return any(getattr(p, "is_lora", False) for p in model.parameters())


@contextlib.contextmanager
def time_measure(context: str = "", suppress_logging: bool = False):
  start = time.perf_counter()
  try:
    yield lambda: time.perf_counter() - start
  finally:
    if not suppress_logging:
      log.info("%s finished in: %.4f seconds", context, time.perf_counter() - start)


def show_hbm_usage(title: str = "") -> None:
  """Logs allocated / reserved / total HBM for every visible GPU."""
  gc.collect()
  if not torch.cuda.is_available():
    log.info("%s - no CUDA device", title)
    return
  for i in range(torch.cuda.device_count()):
    free, total = torch.cuda.mem_get_info(i)
    used = total - free
    log.info("%s - Using %.2f GiB / %.2f GiB (%.3f) on cuda:%d (torch allocated %.2f GiB)", title,
             used / 2**30, total / 2**30, used / total, i, torch.cuda.memory_allocated(i) / 2**30)


def _as_tensor(x) -> torch.Tensor:
  return x if isinstance(x, torch.Tensor) else torch.as_tensor(x, dtype=torch.float32)


@dataclasses.dataclass
class WeightedMetric:
  """A metric reduced as sum / weight, with the division deferred.

  `unreduced_sum` and `denominator` are scalars (tensors or numbers). `eps` is added to the
  denominator, `min_denom` bounds it from below; a zero denominator yields 0, never NaN.
  """

  unreduced_sum: Any
  denominator: Any
  eps: Optional[float] = None
  min_denom: Optional[float] = None

  def compute_scale(self) -> torch.Tensor:
    denom = _as_tensor(self.denominator).float()
    if self.eps is not None:
      denom = denom + self.eps
    if self.min_denom is not None:
      denom = torch.clamp(denom, min=self.min_denom)
    safe = torch.where(denom == 0, torch.ones_like(denom), denom)
    return torch.where(denom == 0, torch.zeros_like(denom), 1.0 / safe)

  def compute(self) -> torch.Tensor:
    s = _as_tensor(self.unreduced_sum)
    return s * self.compute_scale().to(s.device)

  def detach(self) -> "WeightedMetric":
    d = lambda v: v.detach() if isinstance(v, torch.Tensor) else v
    return WeightedMetric(d(self.unreduced_sum), d(self.denominator), self.eps, self.min_denom)


@dataclasses.dataclass
class LossOutput:
  """What a loss function returns: the (unreduced) primary loss and auxiliary metrics.

  The gradient is taken of `primary_loss.unreduced_sum`; the trainer divides by the sum of
  denominators over the micro-batches of an update.
  """

  primary_loss: WeightedMetric
  aux_metrics: Mapping[str, Union[WeightedMetric, Any]] = dataclasses.field(default_factory=dict)
