"""Binary correctness reward for math problems (tunix/utils/math_rewards.py:27-106).

The answer is whatever follows the model's closing thought tag; it scores 1.0 when its last
boxed expression matches any ground truth under the string grader, the symbolic grader or the
special cases of `math_utils`, else 0.0.
"""
from __future__ import annotations

from typing import List, Sequence, Union

from . import math_utils

THOUGHT_DELIMITER_START = "<think>"
THOUGHT_DELIMITER_END = "</think>"


def is_correct(model_answer: str, ground_truth: str) -> bool:
  return (math_utils.grade_answer_mathd(model_answer, ground_truth)
          or math_utils.grade_answer_sympy(model_answer, ground_truth)
          or math_utils.grade_answer_special_handling(model_answer, ground_truth))


def math_reward(prompts: List[str], completions: List[str],
                answer: Sequence[Union[str, float, int, Sequence, None]], **kwargs) -> List[float]:
  del prompts, kwargs
  rewards = []
  for completion, truths in zip(completions, answer):
    if not completion or truths is None:
      rewards.append(0.0)
      continue
    solution = completion.split(THOUGHT_DELIMITER_END)[1] if THOUGHT_DELIMITER_END in completion else completion
    model_answer = math_utils.extract_answer(solution)
    if model_answer is None:
      rewards.append(0.0)
      continue
    if isinstance(truths, (str, float, int)):
      truths = [truths]
    cleaned = []
    for t in truths:
      t = str(t)
      if "\\boxed" in t:
        t = math_utils.extract_answer(t)
      if t is not None:
        cleaned.append(t)
    rewards.append(1.0 if any(is_correct(model_answer, t) for t in cleaned) else 0.0)
  return rewards
