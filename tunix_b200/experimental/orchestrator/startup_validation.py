"""Checks of the run geometry before anything is launched
(tunix/experimental/orchestrator/startup_validation.py:30-164). Every validator returns a list
of messages and all of them are raised together, so one run shows every misconfiguration."""
from __future__ import annotations

from typing import Any, List, Protocol, Sequence, Tuple

from ...rl import utils as rl_utils
from . import worker_registry


class StartupValidationError(ValueError):
  def __init__(self, errors: List[str]):
    self.errors = list(errors)
    super().__init__("startup validation failed:\n  - " + "\n  - ".join(self.errors))


class StartupValidator(Protocol):
  def validate(self, registry: worker_registry.WorkerRegistry, alg_config: Any, training_config: Any) -> List[str]: ...


def _positive(value, name: str, errors: List[str]) -> bool:
  try:
    rl_utils.is_positive_integer(value, name)
    return True
  except ValueError as e:
    errors.append(str(e))
    return False


class RunGeometryValidator:
  """Positive sizes; mini_batch divisible by the group size and by every micro-batch size;
  group size > 1 for group-relative algorithms."""

  def validate(self, registry, alg_config, training_config) -> List[str]:
    errors: List[str] = []
    G = getattr(alg_config, "num_generations", 1)
    mini = getattr(training_config, "mini_batch_size", None)
    _positive(getattr(alg_config, "max_response_length", 1024), "max_response_length", errors)
    g_ok = _positive(G, "num_generations", errors)
    m_ok = _positive(mini, "mini_batch_size", errors)
    if g_ok and m_ok and mini % G != 0:
      errors.append(f"mini_batch_size {mini} is not divisible by num_generations (group_size) {G}")
    if m_ok:
      for name in ("train_micro_batch_size", "rollout_micro_batch_size", "compute_logps_micro_batch_size"):
        v = getattr(training_config, name, None)
        if v is not None and _positive(v, name, errors) and mini % v != 0:
          errors.append(f"mini_batch_size {mini} is not divisible by {name} {v}")
    variant = getattr(alg_config, "algo_variant", "")
    if variant in ("grpo", "gspo-token") and not (isinstance(G, int) and G > 1):
      errors.append(f"num_generations (group_size) must be > 1 for {variant!r}, got {G}")
    return errors


class RoleCoverageValidator:
  """Every role the algorithm needs has at least one registered worker."""

  def __init__(self, required: Sequence[str] = ("actor", "rollout")):
    self.required = tuple(required)

  def validate(self, registry, alg_config, training_config) -> List[str]:
    have = {r.lower() for r in registry.roles()}
    return [f"no worker registered for role {r!r}" for r in self.required if r.lower() not in have]


DEFAULT_VALIDATORS: Tuple[StartupValidator, ...] = (RunGeometryValidator(),)


def validate_startup(registry, alg_config, training_config, *, validators: Sequence[StartupValidator] = DEFAULT_VALIDATORS
                     ) -> None:
  errors: List[str] = []
  for v in validators:
    errors.extend(v.validate(registry, alg_config, training_config))
  if errors:
    raise StartupValidationError(errors)
