"""Thread-safe registry of named functions per category: policy / value loss functions,
advantage estimators, reward managers (tunix/rl/function_registry.py:26-168). Configs refer to
these by string name."""
from __future__ import annotations

import threading
from typing import Any, Callable, Dict, FrozenSet, Iterable, List, Optional

_POLICY_LOSS_FN_CATEGORY = "policy_loss_fn"
_VALUE_LOSS_FN_CATEGORY = "value_loss_fn"
_ADVANTAGE_ESTIMATOR_CATEGORY = "advantage_estimator"
_REWARD_MANAGER_CATEGORY = "reward_manager"


class FunctionRegistry:
  DEFAULT_ALLOWED_CATEGORIES: FrozenSet[str] = frozenset({
      _POLICY_LOSS_FN_CATEGORY, _VALUE_LOSS_FN_CATEGORY, _ADVANTAGE_ESTIMATOR_CATEGORY, _REWARD_MANAGER_CATEGORY})

  def __init__(self, allowed_categories: Optional[Iterable[str]] = None):
    self._allowed_categories = (frozenset(allowed_categories) if allowed_categories is not None
                                else self.DEFAULT_ALLOWED_CATEGORIES)
    self._registry: Dict[str, Dict[str, Callable[..., Any]]] = {c: {} for c in self._allowed_categories}
    self._lock = threading.Lock()

  def _validate_category(self, category: str) -> None:
    if category not in self._allowed_categories:
      raise ValueError(f"Invalid category: '{category}'. Allowed categories are: {sorted(self._allowed_categories)}")

  def register(self, category: str, name: str) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
    self._validate_category(category)

    def decorator(func: Callable[..., Any]) -> Callable[..., Any]:
      with self._lock:
        if name in self._registry[category]:
          raise ValueError(f"'{name}' is already registered in category '{category}'.")
        self._registry[category][name] = func
      return func
    return decorator

  def get(self, category: str, name: str) -> Callable[..., Any]:
    self._validate_category(category)
    with self._lock:
      if name not in self._registry[category]:
        raise LookupError(f"'{name}' not found in category '{category}'. Available: "
                          f"{sorted(self._registry[category])}")
      return self._registry[category][name]

  def list_categories(self) -> List[str]:
    return sorted(self._allowed_categories)

  def list_functions(self, category: str) -> List[str]:
    self._validate_category(category)
    with self._lock:
      return sorted(self._registry[category])


default_registry = FunctionRegistry()


def get_policy_loss_fn(name: str):
  return default_registry.get(_POLICY_LOSS_FN_CATEGORY, name)


def register_policy_loss_fn(name: str):
  return default_registry.register(_POLICY_LOSS_FN_CATEGORY, name)


def get_advantage_estimator(name: str):
  return default_registry.get(_ADVANTAGE_ESTIMATOR_CATEGORY, name)


def register_advantage_estimator(name: str):
  return default_registry.register(_ADVANTAGE_ESTIMATOR_CATEGORY, name)


def get_reward_manager(name: str):
  return default_registry.get(_REWARD_MANAGER_CATEGORY, name)


def register_reward_manager(name: str):
  return default_registry.register(_REWARD_MANAGER_CATEGORY, name)


def get_value_loss_fn(name: str):
  return default_registry.get(_VALUE_LOSS_FN_CATEGORY, name)


def register_value_loss_fn(name: str):
  return default_registry.register(_VALUE_LOSS_FN_CATEGORY, name)
