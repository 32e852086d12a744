"""Metric containers of the experimental trainer (tunix/experimental/metrics/metrics.py).

Values stay on the device, unreduced, until somebody asks for them on the host - a training step then
costs no device-to-host synchronisation for logging."""
from __future__ import annotations

import dataclasses
from typing import Any, Callable, Dict, Optional, Union

import torch

Scalar = Union[torch.Tensor, float, int]


@dataclasses.dataclass
class WeightedMetric:
  """A sum and the weight it has to be divided by (token-weighted loss: sum of token losses, token count).
  `eps` is added to the weight, `min_denom` bounds it from below; both optional."""
  unreduced_sum: Scalar
  denominator: Scalar
  eps: Optional[float] = None
  min_denom: Optional[float] = None

  def compute_scale(self) -> Scalar:
    d = torch.as_tensor(self.denominator, dtype=torch.float32)
    if self.eps is not None:
      d = d + self.eps
    if self.min_denom is not None:
      d = torch.clamp(d, min=self.min_denom)
    return torch.where(d == 0, torch.zeros_like(d), 1.0 / torch.where(d == 0, torch.ones_like(d), d))

  def compute(self) -> Scalar:
    return torch.as_tensor(self.unreduced_sum, dtype=torch.float32) * self.compute_scale()

  def __add__(self, other: "WeightedMetric") -> "WeightedMetric":
    return WeightedMetric(self.unreduced_sum + other.unreduced_sum, self.denominator + other.denominator, self.eps,
                          self.min_denom)


@dataclasses.dataclass
class MetricsBuffer:
  """Metrics of one step (or one micro-batch) in unreduced form, plus how the host should aggregate each."""
  id: Union[int, str, torch.Tensor]
  weighted_metrics: Dict[str, WeightedMetric] = dataclasses.field(default_factory=dict)
  scalar_metrics: Dict[str, Scalar] = dataclasses.field(default_factory=dict)
  aggregation_fns: Dict[str, Callable[[Any], Any]] = dataclasses.field(default_factory=dict)
  mode: str = "train"

  def merge(self, other: "MetricsBuffer") -> "MetricsBuffer":
    """Accumulates another micro-batch of the same step: weighted metrics add, scalars collect into lists."""
    for k, v in other.weighted_metrics.items():
      self.weighted_metrics[k] = self.weighted_metrics[k] + v if k in self.weighted_metrics else v
    for k, v in other.scalar_metrics.items():
      cur = self.scalar_metrics.get(k)
      self.scalar_metrics[k] = [v] if cur is None else (cur + [v] if isinstance(cur, list) else [cur, v])
    self.aggregation_fns.update(other.aggregation_fns)
    return self

  def to_host(self) -> Dict[str, float]:
    """One synchronisation: every value reduced and read back as a Python float."""
    out: Dict[str, float] = {}
    for k, m in self.weighted_metrics.items():
      out[k] = float(torch.as_tensor(m.compute()))
    for k, v in self.scalar_metrics.items():
      vals = v if isinstance(v, list) else [v]
      host = [float(torch.as_tensor(x)) for x in vals]
      fn = self.aggregation_fns.get(k)
      out[k] = float(fn(host)) if fn is not None else host[-1]
    return out
