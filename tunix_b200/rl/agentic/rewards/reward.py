"""Named reward functions `(task, action) -> RewardOutput` (tunix/rl/agentic/rewards/reward.py:30-239)."""
from __future__ import annotations

import ast
import logging
import operator
from typing import Any, Callable, Dict

from . import reward_types

_REGISTRY: Dict[str, Callable[..., reward_types.RewardOutput]] = {}


def register(name: str):
  def wrap(fn):
    if name in _REGISTRY:
      raise ValueError(f"Reward {name} already registered.")
    _REGISTRY[name] = fn
    return fn
  return wrap


def unregister(name: str) -> bool:
  return _REGISTRY.pop(name, None) is not None


def get_reward_fn(name: str):
  return _REGISTRY[name]


@register("exact_match")
def exact_match(task: Dict[str, Any], action: str) -> reward_types.RewardOutput:
  score = 1.0 if action.strip() == str(task.get("ground_truth", "")).strip() else 0.0
  return reward_types.RewardOutput(score, {"exact_match": score})


def combine_rewards(weights: Dict[str, float]):
  """Weighted sum of registered reward functions; metadata dicts are merged."""
  def fn(task: Dict[str, Any], action: str) -> reward_types.RewardOutput:
    total, meta = 0.0, {}
    for name, w in weights.items():
      out = get_reward_fn(name)(task, action)
      total += w * out.reward
      meta.update(out.metadata)
    return reward_types.RewardOutput(total, meta)
  return fn


@register("is_two")
def is_two_reward(task: Dict[str, Any], action: str) -> reward_types.RewardOutput:
  try:
    score = 1.0 if float(action.strip()) == 2.0 else 0.0
  except ValueError:
    score = 0.0
  return reward_types.RewardOutput(score, {"is_two": score})


@register("dummy")
def dummy_reward(task: Dict[str, Any], action: str) -> reward_types.RewardOutput:
  return reward_types.RewardOutput(0.0, {})


_BIN = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.Div: operator.truediv,
        ast.Pow: operator.pow}
_UN = {ast.USub: operator.neg, ast.UAdd: operator.pos}


def _safe_eval(expr: str) -> float:
  """Arithmetic only: numbers, + - * / ** and unary signs."""
  def ev(node):
    if isinstance(node, ast.Constant) and isinstance(node.value, (int, float)) and not isinstance(node.value, bool):
      return node.value
    if isinstance(node, ast.BinOp) and type(node.op) in _BIN:
      return _BIN[type(node.op)](ev(node.left), ev(node.right))
    if isinstance(node, ast.UnaryOp) and type(node.op) in _UN:
      return _UN[type(node.op)](ev(node.operand))
    raise ValueError(f"Unsupported expression element: {type(node).__name__}")
  return float(ev(ast.parse(expr, mode="eval").body))


@register("calculate")
def calculate_reward(task: Dict[str, Any], action: str) -> reward_types.RewardOutput:
  """1.0 when the answer equals the value of the arithmetic expression in task['question']."""
  expression = task.get("question", "").replace("= ?", "").replace("=", "").strip()
  try:
    answer = float(action.replace("The answer is ", "").strip().rstrip("."))
    score = 1.0 if abs(_safe_eval(expression) - answer) < 1e-6 else 0.0
  except Exception as e:
    logging.warning("Failed to calculate reward for task %s and action %s: %s", task, action, e)
    score = 0.0
  return reward_types.RewardOutput(score, {"calculate_correct": score})
