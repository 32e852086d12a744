"""Checkpointing options: when to save, what to keep, sync or async.

Same defaults as tunix/sft/checkpoint_options.py:26-271: continuous policy with at least 180 s
between saves, keep the latest 3, plain integer step directories, asynchronous writes with a
1200 s timeout. `checkpointing_options_from_dict` accepts only `save_interval_steps`,
`max_to_keep`, `enable_async_checkpointing` and `timeout_secs`.
"""
from __future__ import annotations

import dataclasses
import time
from typing import Any, Dict, List, Mapping, Optional

CONFIG_OPTIONS = frozenset(["save_interval_steps", "max_to_keep", "enable_async_checkpointing", "timeout_secs"])


class SaveDecisionPolicy:

  def should_save(self, step: int, last_saved_step: Optional[int], last_save_time: Optional[float]) -> bool:
    raise NotImplementedError


@dataclasses.dataclass(frozen=True)
class ContinuousCheckpointingPolicy(SaveDecisionPolicy):
  """Save whenever no save is in flight and `minimum_interval_secs` have passed."""

  minimum_interval_secs: Optional[float] = None

  def should_save(self, step, last_saved_step, last_save_time):
    if last_save_time is None or not self.minimum_interval_secs:
      return True
    return (time.time() - last_save_time) >= self.minimum_interval_secs


@dataclasses.dataclass(frozen=True)
class FixedIntervalPolicy(SaveDecisionPolicy):
  interval: int

  def should_save(self, step, last_saved_step, last_save_time):
    return step % self.interval == 0


class PreservationPolicy:

  def to_delete(self, steps: List[int]) -> List[int]:
    raise NotImplementedError


@dataclasses.dataclass(frozen=True)
class LatestN(PreservationPolicy):
  n: Optional[int] = None

  def to_delete(self, steps):
    if self.n is None or len(steps) <= self.n:
      return []
    return sorted(steps)[: len(steps) - self.n]


@dataclasses.dataclass(frozen=True)
class AsyncOptions:
  timeout_secs: Optional[int] = 1200


@dataclasses.dataclass(frozen=True)
class TunixCheckpointingOptions:
  save_decision_policy: Optional[SaveDecisionPolicy] = None
  preservation_policy: Optional[PreservationPolicy] = None
  step_name_format: Any = None
  enable_async_checkpointing: Optional[bool] = None
  async_options: Optional[AsyncOptions] = None
  use_ocdbt: bool = False      # array data of each process in one key-value store file instead of a file per array


DEFAULT_CHECKPOINTING_OPTIONS = TunixCheckpointingOptions(
    save_decision_policy=ContinuousCheckpointingPolicy(minimum_interval_secs=180),
    preservation_policy=LatestN(n=3),
    step_name_format=None,
    enable_async_checkpointing=True,
    async_options=AsyncOptions(timeout_secs=1200),
)


def create_checkpointing_options(*, save_decision_policy=None, preservation_policy=None, step_name_format=None,
                                 enable_async_checkpointing=None, async_options=None) -> TunixCheckpointingOptions:
  return TunixCheckpointingOptions(save_decision_policy, preservation_policy, step_name_format,
                                   enable_async_checkpointing, async_options)


def resolve_checkpointing_defaults(options: Any = None) -> TunixCheckpointingOptions:
  """Fills unset fields from the defaults. Objects with the legacy fields
  `save_interval_steps` / `max_to_keep` are understood too."""
  d = DEFAULT_CHECKPOINTING_OPTIONS
  if options is None:
    return d
  save_policy = getattr(options, "save_decision_policy", None)
  if save_policy is None and getattr(options, "save_interval_steps", None):
    save_policy = FixedIntervalPolicy(int(options.save_interval_steps))
  pres = getattr(options, "preservation_policy", None)
  if pres is None and getattr(options, "max_to_keep", None):
    pres = LatestN(int(options.max_to_keep))
  en = getattr(options, "enable_async_checkpointing", None)
  ao = getattr(options, "async_options", None)
  return TunixCheckpointingOptions(
      save_decision_policy=save_policy or d.save_decision_policy,
      preservation_policy=pres or d.preservation_policy,
      step_name_format=getattr(options, "step_name_format", None),
      enable_async_checkpointing=d.enable_async_checkpointing if en is None else en,
      async_options=ao or d.async_options,
      use_ocdbt=bool(getattr(options, "use_ocdbt", False)),
  )


def checkpointing_options_from_dict(cfg: Optional[Mapping[str, Any]]) -> Optional[TunixCheckpointingOptions]:
  """Builds options from a config mapping; unknown keys are an error."""
  if not cfg:
    return None
  unknown = set(cfg) - CONFIG_OPTIONS
  if unknown:
    raise ValueError(f"Unsupported checkpointing options: {sorted(unknown)}. Supported: {sorted(CONFIG_OPTIONS)}")
  save = FixedIntervalPolicy(int(cfg["save_interval_steps"])) if cfg.get("save_interval_steps") else None
  keep = LatestN(int(cfg["max_to_keep"])) if cfg.get("max_to_keep") else None
  ao = AsyncOptions(int(cfg["timeout_secs"])) if cfg.get("timeout_secs") else None
  return TunixCheckpointingOptions(save, keep, None, cfg.get("enable_async_checkpointing"), ao)
