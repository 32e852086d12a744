"""verl-style GSM8K scorer: `compute_score(solution_str, ground_truth)` on `#### <number>`
answers (tunix/cli/reward_fn/gsm8k_verl.py:21-76). Used through the `verl_compatible` adapter."""
from __future__ import annotations

import re
from typing import Optional

_SOLUTION_CLIP_CHARS = 300
_STRICT = re.compile(r"#### (\-?[0-9\.\,]+)")
_FLEX = re.compile(r"(\-?[0-9\.\,]+)")


def extract_solution(solution_str: str, method: str = "strict") -> Optional[str]:
  """Only the last 300 characters are searched. strict: last `#### n`; flexible: last number."""
  assert method in ("strict", "flexible")
  tail = solution_str[-_SOLUTION_CLIP_CHARS:]
  if method == "strict":
    found = _STRICT.findall(tail)
    return found[-1].replace(",", "").replace("$", "") if found else None
  found = _FLEX.findall(tail)
  pick = None
  for pick in reversed(found):
    if pick not in ("", "."):
      break
  return pick


def compute_score(solution_str: str, ground_truth: str, method: str = "strict", format_score: float = 0.0,
                  score: float = 1.0) -> float:
  answer = extract_solution(solution_str, method)
  if answer is None:
    return 0
  return score if answer == ground_truth else format_score
