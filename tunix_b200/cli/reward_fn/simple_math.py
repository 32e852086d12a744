"""Format + exact-number rewards for simple arithmetic tasks
(tunix/cli/reward_fn/simple_math.py:23-70)."""
from __future__ import annotations

import re
from typing import List

reasoning_start, reasoning_end = "<reasoning>", "</reasoning>"
solution_start, solution_end = "<answer>", "</answer>"
match_format = re.compile(r"^[\s]{0,}" + reasoning_start + r".+?" + reasoning_end + r".*?" + solution_start +
                          r"(.+?)" + solution_end + r"[\s]{0,}$", flags=re.MULTILINE | re.DOTALL)
_number = re.compile(solution_start + r".*?([\d\.]{1,})", flags=re.MULTILINE | re.DOTALL)


def check_format(prompts, completions, r: float = 0.1, **kwargs) -> List[float]:
  return [r if match_format.search(c) else 0 for c in completions]


def check_answer(prompts, completions, answer, r: float = 1, **kwargs) -> List[float]:
  out = []
  for c, a in zip(completions, answer):
    m = _number.search(c)
    if m is None:
      out.append(0)
      continue
    try:
      out.append(r if float(m.group(1).strip()) == float(str(a).strip()) else 0.0)
    except ValueError:
      out.append(0)
  return out
