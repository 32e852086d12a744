"""GSM8K pieces of the distributed GRPO example (tunix/experimental/examples/math_gsm8k_dist/gsm8k.py): the prompt
template, answer extraction and rewards, task loading, and a single-step environment and agent registered by name
for rollout workers that run episodes instead of plain completions.

Tasks come from a local JSON-lines file in the dataset's own format ({"question": ..., "answer": "... #### 72"}) or,
with no file, from a generator of small arithmetic word problems, so the example runs with no dataset on disk.
"""
from __future__ import annotations

import json
import random
import re
from typing import Any, Callable, Dict, Iterator, List, Optional, Tuple

from ....rl.agentic.agents import agent_types, base_agent
from ....rl.agentic.environments import base_environment
from ...rl.agentic import registry

GSM8K_ENV_NAME = "gsm8kenv"
GSM8K_AGENT_NAME = "gsm8kagent"

PROMPT_TEMPLATE = (
    "Solve the following math problem.\n"
    "First, put your detailed step-by-step reasoning process inside <reasoning>...</reasoning> tags.\n"
    "Then, put your final numerical answer inside <answer>\\boxed{{}}</answer> tags.\n\n"
    "Problem: {question}\n<reasoning>\n")

_BOXED = re.compile(r"\\boxed\{\s*([^{}]+?)\s*\}")
_TAGGED = re.compile(r"<answer>\s*(.*?)\s*</answer>", re.S)
_NUMBER = re.compile(r"-?\d[\d,]*(?:\.\d+)?")


def _canonical(number: str) -> str:
  number = number.replace(",", "").strip().rstrip(".")
  if re.fullmatch(r"-?\d+\.0+", number):
    number = number.split(".")[0]
  return number


def extract_answer(text: str) -> Optional[str]:
  """The final answer of a completion: the last \\boxed{...}, else the last <answer> tag; None when neither holds a
  number. (A bare number elsewhere in the text is reasoning, not an answer.)"""
  for pattern in (_BOXED, _TAGGED):
    found = pattern.findall(text or "")
    if found:
      numbers = _NUMBER.findall(found[-1])
      if numbers:
        return _canonical(numbers[-1])
  return None


def gold_of(answer_field: str) -> str:
  """'... #### 72' -> '72' (the dataset's convention); a bare number passes through."""
  return _canonical(answer_field.rsplit("####", 1)[-1])


def make_reward_fn(mode: str = "answer") -> Callable[[Any], float]:
  """Reward of one trajectory item whose metadata carries `gold_answer` and `completion_text`.
  "answer": 1 for the right final answer, plus 0.1 for using the answer format at all;
  "contains": 1 when the gold answer appears anywhere (what the environment below scores);
  "length": a smoke-test signal that needs no correct answers - shorter completions score higher."""
  def answer(item: Any) -> float:
    md = item.metadata or {}
    got = extract_answer(md.get("completion_text", ""))
    return (1.0 if got is not None and got == str(md.get("gold_answer")) else 0.0) + (0.1 if got is not None else 0.0)

  def contains(item: Any) -> float:
    md = item.metadata or {}
    gold = str(md.get("gold_answer", ""))
    return 1.0 if gold and gold in md.get("completion_text", "") else 0.0

  def length(item: Any) -> float:
    return 1.0 / (1.0 + len(item.completion_tokens))
  try:
    return {"answer": answer, "contains": contains, "length": length}[mode]
  except KeyError:
    raise ValueError(f"unknown reward mode {mode!r}; choose answer, contains or length") from None


def synthetic_tasks(count: int, seed: int = 0) -> Iterator[Tuple[str, str]]:
  rng = random.Random(seed)
  names = ["Natalia", "Weng", "Betty", "Julie", "James", "Albert"]
  things = ["clips", "pages", "apples", "stickers", "laps", "coins"]
  for _ in range(count):
    who, what, a, b = rng.choice(names), rng.choice(things), rng.randint(2, 60), rng.randint(2, 9)
    kind = rng.randrange(3)
    if kind == 0:
      yield f"{who} had {a} {what} and got {b} more. How many {what} does {who} have now?", str(a + b)
    elif kind == 1:
      yield f"{who} collects {a} {what} a day for {b} days. How many {what} is that altogether?", str(a * b)
    else:
      yield (f"{who} sold {2 * a} {what} in April and half as many in May. How many {what} did {who} sell "
             f"altogether?"), str(3 * a)


def load_tasks(path: Optional[str], count: int, seed: int = 0) -> List[Tuple[str, str]]:
  if not path:
    return list(synthetic_tasks(count, seed))
  tasks = []
  with open(path, "r", encoding="utf-8") as f:
    for line in f:
      if line.strip():
        row = json.loads(line)
        tasks.append((row["question"], gold_of(str(row["answer"]))))
      if len(tasks) >= count:
        break
  return tasks


def prompt_items(tasks: List[Tuple[str, str]], generation_kwargs: Dict[str, Any], agentic: bool = False
                 ) -> List[Dict[str, Any]]:
  """Dataset rows for the RL program: the gold answer rides in the metadata and comes back on every sample."""
  rows = []
  for index, (question, gold) in enumerate(tasks):
    metadata: Dict[str, Any] = {"gold_answer": gold}
    if agentic:
      metadata["env_config"] = {"env_type": GSM8K_ENV_NAME, "agent_type": GSM8K_AGENT_NAME,
                                "prompt": PROMPT_TEMPLATE.format(question=question), "gold_answer": gold}
    rows.append({"prompt_id": f"gsm8k_{index:05d}", "prompt": PROMPT_TEMPLATE.format(question=question),
                 "metadata": metadata, "generation_kwargs": dict(generation_kwargs), "max_turns": 1})
  return rows


class _OneShot(base_environment.BaseTaskEnv):
  """A task that ends with the first action; subclasses say how an action scores."""

  def __init__(self, task: Dict[str, Any], group_id: str = "", pair_index: int = 0, **kwargs: Any):
    kwargs.setdefault("max_steps", 1)
    super().__init__(task=task, group_id=group_id, pair_index=pair_index, **kwargs)

  def score(self, said: str) -> Tuple[float, Dict[str, Any]]:
    raise NotImplementedError

  def _step_impl(self, action: Any) -> base_environment.EnvStepResult:
    said = str(getattr(action, "action", action))
    reward, info = self.score(said)
    return base_environment.EnvStepResult(observation={"answer": said, **info.pop("show", {})}, reward=reward,
                                          done=True, info=info)


@registry.register_env(GSM8K_ENV_NAME)
class GSM8KEnv(_OneShot):
  """The action is the model's answer text; reward 1 when it contains the gold answer (the lenient check: rollout
  workers that want the strict one score `extract_answer` through `make_reward_fn("answer")` on the control plane)."""

  def __init__(self, prompt: str = "", gold_answer: str = "", policy_version: int = 0, **kwargs: Any):
    self.gold = str(gold_answer)
    super().__init__({"prompts": prompt, "gold_answer": self.gold, "policy_version": policy_version}, **kwargs)

  def _initial_observation(self) -> Dict[str, str]:
    return {"prompts": self.task["prompts"]}

  def score(self, said: str) -> Tuple[float, Dict[str, Any]]:
    hit = self.gold != "" and self.gold in said
    return float(hit), {"correct": hit, "show": {"gold_answer": self.gold}}


@registry.register_agent(GSM8K_AGENT_NAME)
class GSM8KAgent(base_agent.ConversationAgentBase):
  """Hands the model's text to the environment unchanged and keeps it in the conversation."""

  name = GSM8K_AGENT_NAME
  SYSTEM_PROMPT = "Solve the math problem. Return the final numeric answer clearly."

  def __init__(self):
    super().__init__(self.SYSTEM_PROMPT)

  def update_from_model(self, response: str, **kwargs: Any) -> agent_types.Action:
    step = agent_types.Step(model_response=response, thought="", action=agent_types.Action(action=response))
    self.trajectory.steps.append(step)
    self.chat_completions.append({"role": "assistant", "content": response})
    return step.action
