"""Profiler window around training steps.

Starts a `torch.profiler` trace (CPU + CUDA activities, Chrome/Perfetto-loadable output) at
step `initial_step + skip_first_n_steps` and stops it `profiler_steps` later; rank 0 only; a
class-level lock keeps a single profiler active per process (tunix/sft/profiler.py:25-166).
"""
from __future__ import annotations

import dataclasses
import logging
import os
import threading
from typing import Optional

log = logging.getLogger(__name__)


@dataclasses.dataclass(frozen=True)
class ProfilerOptions:
  log_dir: str
  skip_first_n_steps: int
  profiler_steps: int
  set_profile_options: bool = True
  host_tracer_level: int = 2     # >= 2 also records memory events
  python_tracer_level: int = 1   # >= 1 records Python stacks
  max_num_hosts: Optional[int] = None


class Profiler:
  _lock = threading.Lock()
  _is_active: bool = False

  def __init__(self, initial_step: int, max_step: Optional[int], profiler_options: Optional[ProfilerOptions]):
    if int(os.environ.get("RANK", "0")) != 0 or profiler_options is None:
      self._do_not_profile = True
      return
    self._profiler_options = profiler_options
    self._do_not_profile = False
    self._output_path = profiler_options.log_dir
    self._first_profile_step = initial_step + profiler_options.skip_first_n_steps
    self._last_profile_step = self._set_last_profile_step(profiler_options.profiler_steps, max_step)
    if self._first_profile_step >= self._last_profile_step:
      raise ValueError(f"First profile step {self._first_profile_step} cannot be greater than the last profile "
                       f"step {self._last_profile_step}.")
    self._started_by_this_instance = False
    self._prof = None

  def _set_last_profile_step(self, profiler_steps: int, max_step: Optional[int]) -> int:
    last = self._first_profile_step + profiler_steps
    if max_step is not None:
      last = min(last, max_step)
    return last

  def _start_trace(self) -> None:
    import torch
    o = self._profiler_options
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
      acts.append(torch.profiler.ProfilerActivity.CUDA)
    os.makedirs(self._output_path, exist_ok=True)
    kwargs = {}
    if o.set_profile_options:
      kwargs = dict(profile_memory=o.host_tracer_level >= 2, with_stack=o.python_tracer_level >= 1)
    self._prof = torch.profiler.profile(
        activities=acts, on_trace_ready=torch.profiler.tensorboard_trace_handler(self._output_path), **kwargs)
    self._prof.start()

  def _stop_trace(self) -> None:
    if self._prof is not None:
      self._prof.stop()
      self._prof = None

  def maybe_activate(self, step: int) -> None:
    if self._do_not_profile or step != self._first_profile_step:
      return
    with Profiler._lock:
      if Profiler._is_active:
        log.warning("A profiler is already active; skipping activation at step %d.", step)
        return
      log.info("Starting profiler at step %d.", step)
      self._start_trace()
      Profiler._is_active = True
      self._started_by_this_instance = True

  def maybe_deactivate(self, step: int) -> None:
    if self._do_not_profile or step != self._last_profile_step:
      return
    with Profiler._lock:
      if not self._started_by_this_instance:
        return
      log.info("Stopping profiler at step %d.", step)
      self._stop_trace()
      Profiler._is_active = False
      self._started_by_this_instance = False
