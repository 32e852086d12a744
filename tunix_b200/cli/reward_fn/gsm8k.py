"""GSM8K reward functions for `<reasoning>…</reasoning><answer>…</answer>` completions
(scoring table of tunix/cli/reward_fn/gsm8k.py:33-145). Every public function here is picked
up by `HyperParameters.obtain_reward_fn` and has the signature
`fn(prompts, completions, **dataset_columns) -> list of float`."""
from __future__ import annotations

import logging
import os
import re
from typing import List, Optional

reasoning_start, reasoning_end = "<reasoning>", "</reasoning>"
solution_start, solution_end = "<answer>", "</answer>"
_TAGS = (reasoning_start, reasoning_end, solution_start, solution_end)

match_format = re.compile(
    re.escape(reasoning_start) + r".+?" + re.escape(reasoning_end) + r".*?" + re.escape(solution_start) +
    r"(.+?)(?:" + re.escape(solution_end) + r"|$)", flags=re.MULTILINE | re.DOTALL)
_first_number = re.compile(re.escape(solution_start) + r".*?([\d\.]{1,})", flags=re.MULTILINE | re.DOTALL)


def _clean(x) -> str:
  return str(x).strip().replace(",", "")


def match_format_exactly(prompts, completions, **kwargs) -> List[float]:
  """3 points when the completion has the full reasoning + answer structure."""
  return [3.0 if match_format.search(c) else 0 for c in completions]


def match_format_approximately(prompts, completions, **kwargs) -> List[float]:
  """+0.5 for each of the four tags that occurs exactly once, -0.5 otherwise."""
  return [sum(0.5 if c.count(tag) == 1 else -0.5 for tag in _TAGS) for c in completions]


def _grade(guess: Optional[str], truth: str) -> float:
  if guess is None:
    return 0
  if guess == truth:
    return 3.0
  try:
    g, t = float(guess), float(truth)
  except ValueError:
    return -0.5
  if g == t:
    return 3.0
  if t == 0:
    return -1.0 if g != 0 else 0.0
  ratio = g / t
  if 0.9 <= ratio <= 1.1:
    return 0.5
  if 0.8 <= ratio <= 1.2:
    return 0.25
  return -1.0


def check_answer(prompts, completions, answer, **kwargs) -> List[float]:
  """Exact match 3, within 10 % 0.5, within 20 % 0.25, wrong -1, unparsable -0.5, no answer 0."""
  truths = [_clean(a) for a in answer]
  if os.environ.get("LOG_GRPO_ROLLOUT", "0") == "1":
    logging.info("GRPO rollout prompts=%r completions=%r answers=%r", prompts, completions, truths)
  out = []
  for c, t in zip(completions, truths):
    m = match_format.search(c)
    out.append(_grade(_clean(m.group(1)) if m else None, t))
  return out


def check_numbers(prompts, completions, answer, **kwargs) -> List[float]:
  """1.5 when the first number after `<answer>` equals the gold answer."""
  out = []
  for c, a in zip(completions, answer):
    m = _first_number.search(c)
    if m is None:
      out.append(0)
      continue
    try:
      out.append(1.5 if float(_clean(m.group(1))) == float(_clean(a)) else 0.0)
    except ValueError:
      out.append(0)
  return out
