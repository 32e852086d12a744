"""Named functions that configs refer to by string: policy / value loss functions, advantage estimators, reward
managers (tunix/rl/function_registry.py:26-168).

A `FunctionRegistry` is a set of *categories*, each a name -> callable table. Entries are immutable once added
(registering a name twice is an error), tables are copy-on-write under one lock so that lookups - which happen on the
training path - take no lock, and the category-specific helpers at the bottom (`register_policy_loss_fn`, ...) are
generated from one list instead of being spelled out four times.
"""
from __future__ import annotations

import threading
from typing import Any, Callable, Dict, FrozenSet, Iterable, List, Mapping, Optional

Fn = Callable[..., Any]

_POLICY_LOSS_FN_CATEGORY = "policy_loss_fn"
_VALUE_LOSS_FN_CATEGORY = "value_loss_fn"
_ADVANTAGE_ESTIMATOR_CATEGORY = "advantage_estimator"
_REWARD_MANAGER_CATEGORY = "reward_manager"
_BUILT_IN = (_POLICY_LOSS_FN_CATEGORY, _VALUE_LOSS_FN_CATEGORY, _ADVANTAGE_ESTIMATOR_CATEGORY, _REWARD_MANAGER_CATEGORY)


class FunctionRegistry:
  DEFAULT_ALLOWED_CATEGORIES: FrozenSet[str] = frozenset(_BUILT_IN)

  def __init__(self, allowed_categories: Optional[Iterable[str]] = None):
    self._allowed_categories = (self.DEFAULT_ALLOWED_CATEGORIES if allowed_categories is None
                                else frozenset(allowed_categories))
    self._tables: Mapping[str, Mapping[str, Fn]] = {c: {} for c in self._allowed_categories}
    self._write = threading.Lock()

  def _table(self, category: str) -> Mapping[str, Fn]:
    try:
      return self._tables[category]
    except KeyError:
      raise ValueError(f"Invalid category: '{category}'. Allowed categories are: "
                       f"{sorted(self._allowed_categories)}") from None

  def add(self, category: str, name: str, func: Fn) -> Fn:
    self._table(category)                                   # validates before taking the lock
    with self._write:
      table = self._tables[category]
      if name in table:
        raise ValueError(f"'{name}' is already registered in category '{category}'.")
      self._tables = {**self._tables, category: {**table, name: func}}
    return func

  def register(self, category: str, name: str) -> Callable[[Fn], Fn]:
    """Decorator form of `add`."""
    self._table(category)
    return lambda func: self.add(category, name, func)

  def get(self, category: str, name: str) -> Fn:
    table = self._table(category)
    if name not in table:
      raise LookupError(f"'{name}' not found in category '{category}'. Available: {sorted(table)}")
    return table[name]

  def list_categories(self) -> List[str]:
    return sorted(self._allowed_categories)

  def list_functions(self, category: str) -> List[str]:
    return sorted(self._table(category))


default_registry = FunctionRegistry()


def _helpers(category: str):
  def getter(name: str) -> Fn:
    return default_registry.get(category, name)

  def registrar(name: str) -> Callable[[Fn], Fn]:
    return default_registry.register(category, name)
  getter.__doc__ = f"The `{category}` registered under `name` in the default registry."
  registrar.__doc__ = f"Decorator: registers a `{category}` under `name` in the default registry."
  return getter, registrar


get_policy_loss_fn, register_policy_loss_fn = _helpers(_POLICY_LOSS_FN_CATEGORY)
get_value_loss_fn, register_value_loss_fn = _helpers(_VALUE_LOSS_FN_CATEGORY)
get_advantage_estimator, register_advantage_estimator = _helpers(_ADVANTAGE_ESTIMATOR_CATEGORY)
get_reward_manager, register_reward_manager = _helpers(_REWARD_MANAGER_CATEGORY)
