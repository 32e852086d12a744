"""Named reward functions `(task, action) -> RewardOutput` (tunix/rl/agentic/rewards/reward.py:30-239).

Most rewards here are yes/no checks, so they are written as predicates and lifted by `@check(name, metric)`
into reward functions that return 1.0 / 0.0 and report the same value under `metric` - a predicate that raises
counts as "no". `combine_rewards` builds a weighted sum of registered rewards. The arithmetic reward needs the
value of an expression written by a dataset, which must never be `eval`-ed: `arithmetic()` is a small
recursive-descent evaluator over numbers, `+ - * / **`, unary signs and parentheses, nothing else.
"""
from __future__ import annotations

import logging
import re
from typing import Any, Callable, Dict, Iterator, List, Tuple

from . import reward_types

RewardFn = Callable[..., reward_types.RewardOutput]
_REGISTRY: Dict[str, RewardFn] = {}


# ---------------------------------------------------------------------------- registry
def register(name: str) -> Callable[[RewardFn], RewardFn]:
  def add(fn: RewardFn) -> RewardFn:
    if name in _REGISTRY:
      raise ValueError(f"Reward {name} already registered.")
    _REGISTRY[name] = fn
    return fn
  return add


def unregister(name: str) -> bool:
  return _REGISTRY.pop(name, None) is not None


def get_reward_fn(name: str) -> RewardFn:
  return _REGISTRY[name]


def check(name: str, metric: str) -> Callable[[Callable[[Dict[str, Any], str], bool]], RewardFn]:
  """Registers a predicate as a 0/1 reward that reports its value as `metric`."""
  def lift(predicate: Callable[[Dict[str, Any], str], bool]) -> RewardFn:
    def reward(task: Dict[str, Any], action: str) -> reward_types.RewardOutput:
      try:
        score = float(bool(predicate(task, action)))
      except Exception as e:      # noqa: BLE001 - an answer that cannot be checked is a wrong answer
        logging.warning("Failed to calculate reward for task %s and action %s: %s", task, action, e)
        score = 0.0
      return reward_types.RewardOutput(score, {metric: score})
    reward.__name__, reward.__doc__ = predicate.__name__, predicate.__doc__
    return register(name)(reward)
  return lift


def combine_rewards(weights: Dict[str, float]) -> RewardFn:
  """Weighted sum of registered reward functions; their metadata dicts are merged."""
  def combined(task: Dict[str, Any], action: str) -> reward_types.RewardOutput:
    parts = [(w, get_reward_fn(name)(task, action)) for name, w in weights.items()]
    merged: Dict[str, Any] = {}
    for _, out in parts:
      merged.update(out.metadata)
    return reward_types.RewardOutput(sum(w * out.reward for w, out in parts), merged)
  return combined


# ---------------------------------------------------------------------------- arithmetic without eval
_TOKEN = re.compile(r"\s*(?:(\d+\.?\d*(?:[eE][+-]?\d+)?|\.\d+)|(\*\*|[-+*/()]))")


def _tokens(text: str) -> Iterator[Tuple[str, str]]:
  pos, text = 0, text.rstrip()
  while pos < len(text):
    m = _TOKEN.match(text, pos)
    if m is None:
      raise ValueError(f"Unsupported expression element at {text[pos:pos + 12]!r}")
    pos = m.end()
    yield ("num", m.group(1)) if m.group(1) is not None else ("op", m.group(2))


def arithmetic(text: str) -> float:
  """Value of an arithmetic expression. Grammar: sum := term (('+'|'-') term)*; term := unary (('*'|'/') unary)*;
  unary := ('+'|'-') unary | power; power := atom ('**' unary)?; atom := number | '(' sum ')'."""
  toks: List[Tuple[str, str]] = list(_tokens(text))
  at = 0

  def peek() -> str:
    return toks[at][1] if at < len(toks) and toks[at][0] == "op" else ""

  def atom() -> float:
    nonlocal at
    if at >= len(toks):
      raise ValueError("expression ends early")
    kind, val = toks[at]
    at += 1
    if kind == "num":
      return float(val)
    if val == "(":
      inner = total()
      if peek() != ")":
        raise ValueError("missing ')'")
      at += 1
      return inner
    raise ValueError(f"unexpected {val!r}")

  def unary() -> float:
    nonlocal at
    if peek() in ("+", "-"):
      sign = -1.0 if peek() == "-" else 1.0
      at += 1
      return sign * unary()
    base = atom()
    if peek() == "**":
      at += 1
      return base ** unary()
    return base

  def term() -> float:
    nonlocal at
    val = unary()
    while peek() in ("*", "/"):
      op = peek()
      at += 1
      rhs = unary()
      val = val * rhs if op == "*" else val / rhs
    return val

  def total() -> float:
    nonlocal at
    val = term()
    while peek() in ("+", "-"):
      op = peek()
      at += 1
      rhs = term()
      val = val + rhs if op == "+" else val - rhs
    return val

  out = total()
  if at != len(toks):
    raise ValueError(f"unexpected {toks[at][1]!r}")
  return out


_safe_eval = arithmetic


# ---------------------------------------------------------------------------- the stock rewards
@check("exact_match", "exact_match")
def exact_match(task: Dict[str, Any], action: str) -> bool:
  """The answer equals task['ground_truth'] up to surrounding white space."""
  return action.strip() == str(task.get("ground_truth", "")).strip()


@check("is_two", "is_two")
def is_two_reward(task: Dict[str, Any], action: str) -> bool:
  """The answer is the number 2."""
  return float(action.strip()) == 2.0


@register("dummy")
def dummy_reward(task: Dict[str, Any], action: str) -> reward_types.RewardOutput:
  return reward_types.RewardOutput(0.0, {})


@check("calculate", "calculate_correct")
def calculate_reward(task: Dict[str, Any], action: str) -> bool:
  """The answer ("The answer is 14.") equals the value of the arithmetic expression in task['question']
  ("2 * (3 + 4) = ?")."""
  expression = task.get("question", "").replace("= ?", "").replace("=", "").strip()
  answer = float(action.replace("The answer is ", "").strip().rstrip("."))
  return abs(arithmetic(expression) - answer) < 1e-6
