"""tqdm progress bar showing the latest logged metrics (tunix/sft/progress_bar.py:21-110).

The postfix shows one entry per (mode, metric), named `<prefix>_<mode>_<metric>`, with all training entries before
the evaluation ones so that the line does not reshuffle when an evaluation happens. The bar draws only where somebody
can see it redraw: a terminal on stderr or a notebook; in a log file it would be one line per refresh.
"""
from __future__ import annotations

import logging
import sys
from typing import Any, Dict, List, Optional

try:
  from tqdm.auto import tqdm
except Exception:  # pragma: no cover
  tqdm = None

log = logging.getLogger(__name__)
_MODE_ORDER = ("train", "eval")
_QUIETLY_ABSENT = frozenset({"learning_rate"})       # not every optimizer reports one


def _is_in_ipython() -> bool:
  try:
    from IPython import get_ipython                 # type: ignore
    return get_ipython() is not None
  except Exception:  # noqa: BLE001 - no IPython, no notebook
    return False


class ProgressBar:

  def __init__(self, metrics_logger: Any, initial_steps: int, max_steps: int, description: Optional[str] = "Training",
               metrics_prefix: str = ""):
    self.metrics_logger = metrics_logger
    self.metrics_prefix = metrics_prefix
    self.initial_steps, self.max_steps, self.description = initial_steps, max_steps, description
    self.metrics: Dict[str, float] = {}
    self._by_mode: Dict[str, Dict[str, float]] = {}
    self.tqdm_bar = None
    if tqdm is not None:
      self.tqdm_bar = tqdm(total=max_steps, initial=initial_steps, desc=description, unit="step", dynamic_ncols=True,
                           leave=True, disable=not (_is_in_ipython() or sys.stderr.isatty()))

  def _update_metric(self, metric_name: str, mode: Any, ndigits: int = 3) -> None:
    mode_name = str(getattr(mode, "value", mode))
    if not self.metrics_logger.metric_exists(self.metrics_prefix, metric_name, mode):
      if metric_name not in _QUIETLY_ABSENT:
        log.warning("Metric %s not found for mode %s. Not showing it.", metric_name, mode_name)
      return
    value = self.metrics_logger.get_metric(self.metrics_prefix, metric_name, mode)
    self._by_mode.setdefault(mode_name, {})[f"{self.metrics_prefix}_{mode_name}_{metric_name}"] = round(float(value), ndigits)
    ordered = [m for m in _MODE_ORDER if m in self._by_mode] + [m for m in self._by_mode if m not in _MODE_ORDER]
    self.metrics = {k: v for m in ordered for k, v in self._by_mode[m].items()}

  def update_metrics(self, metric_names: List[str], mode: Any, ndigits: int = 3) -> None:
    for name in metric_names:
      self._update_metric(name, mode, ndigits)

  def update(self, n: int = 1) -> None:
    if self.tqdm_bar is not None:
      if self.metrics:
        self.tqdm_bar.set_postfix(self.metrics)
      self.tqdm_bar.update(n)

  def close(self) -> None:
    if self.tqdm_bar is not None:
      self.tqdm_bar.close()
      self.tqdm_bar = None
