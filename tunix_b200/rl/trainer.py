"""`PeftTrainer` specialised for RL: logs the aux metrics of the RL loss, shows selected ones in
the progress bar, and stores `global_step` / `role` in checkpoint metadata so a resumed run
continues at the right global step (tunix/rl/trainer.py:29-115)."""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

import numpy as np

from ..sft import peft_trainer
from ..sft.metrics_logger import Mode


class Trainer(peft_trainer.PeftTrainer):

  def __init__(self, model, optimizer, training_config, custom_checkpoint_metadata_fn: Optional[Callable[[], Dict[str, Any]]] = None,
               metrics_logger=None, perf_tracer=None, perf_tracer_v2=None):
    super().__init__(model, optimizer, training_config, metrics_logger, perf_tracer, perf_tracer_v2)
    self.rl_metrics_to_log: Dict[str, Any] = {}
    self.tqdm_metrics_to_display: List[Any] = []
    self.custom_checkpoint_metadata_fn = custom_checkpoint_metadata_fn

  def with_rl_metrics_to_log(self, rl_metrics_to_log: Dict[str, Any]):
    """`{metric name in aux: reducer}`: which aux metrics are logged (under the same name)."""
    self.rl_metrics_to_log = rl_metrics_to_log
    return self

  def with_tqdm_metrics_to_display(self, tqdm_metrics_to_display: List[Any]):
    self.tqdm_metrics_to_display = tqdm_metrics_to_display
    return self

  def custom_checkpoint_metadata(self) -> Dict[str, Any]:
    return self.custom_checkpoint_metadata_fn() if self.custom_checkpoint_metadata_fn else {}

  def restored_global_step(self) -> int:
    return int((self._restored_custom_metadata or {}).get("global_step", 0))

  def _post_process_train_step(self, aux: Any) -> None:
    if not isinstance(aux, dict):
      return
    assert self._buffered_train_metrics is not None
    for name, op in self.rl_metrics_to_log.items():
      if name not in aux:
        continue
      d = self._buffered_train_metrics.additional_metrics
      if name not in d:        # LossOutput aux metrics were buffered already by the base class
        d[name] = ([aux[name]], op)

  def _post_process_eval_step(self, aux: Any) -> None:
    if not isinstance(aux, dict):
      return
    assert self._buffered_eval_metrics is not None
    for name, op in self.rl_metrics_to_log.items():
      if name in aux and name not in self._buffered_eval_metrics.additional_metrics:
        self._buffered_eval_metrics.additional_metrics[name] = ([aux[name]], op)

  def _get_additional_tqdm_metrics(self) -> List[str]:
    out = []
    for m in self.tqdm_metrics_to_display:
      out.append(m() if callable(m) else m)
    return out

  @property
  def _tqdm_train_metrics(self) -> List[str]:
    return ["loss", "perplexity", "learning_rate"] + self._get_additional_tqdm_metrics()
