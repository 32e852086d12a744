"""tqdm progress bar showing the latest logged metrics (tunix/sft/progress_bar.py:21-110)."""
from __future__ import annotations

from typing import Any, List, Optional

try:
  from tqdm.auto import tqdm
except Exception:  # pragma: no cover
  tqdm = None


class ProgressBar:

  def __init__(self, metrics_logger: Any, initial_steps: int, max_steps: int, description: Optional[str] = "Training",
               metrics_prefix: str = ""):
    self.metrics_logger = metrics_logger
    self.metrics_prefix = metrics_prefix
    self.metrics = {}
    self.tqdm_bar = None
    if tqdm is not None:
      self.tqdm_bar = tqdm(total=max_steps, initial=initial_steps, desc=description, unit="step", dynamic_ncols=True,
                           leave=True)

  def _update_metric(self, metric_name: str, mode: Any, ndigits: int = 3) -> None:
    if not self.metrics_logger.metric_exists(self.metrics_prefix, metric_name, mode):
      return
    value = self.metrics_logger.get_metric(self.metrics_prefix, metric_name, mode)
    self.metrics[f"{mode}_{metric_name}"] = round(float(value), ndigits)

  def update_metrics(self, metric_names: List[str], mode: Any, ndigits: int = 3) -> None:
    for name in metric_names:
      self._update_metric(name, mode, ndigits)
    if self.tqdm_bar is not None:
      self.tqdm_bar.set_postfix(self.metrics)

  def update(self, n: int = 1) -> None:
    if self.tqdm_bar is not None:
      self.tqdm_bar.update(n)

  def close(self) -> None:
    if self.tqdm_bar is not None:
      self.tqdm_bar.close()
      self.tqdm_bar = None
