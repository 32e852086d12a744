"""FrozenLake as a text environment.

The agent sees the board as text (`P` player, `_` ice, `O` hole, `G` goal) and answers with one
of Up / Down / Left / Right each turn; reaching the goal gives reward 1, falling into a hole or
running out of steps gives 0. Boards are generated from a seed and are always solvable.
`FrozenLakeEnv` follows `BaseTaskEnv`; `FrozenLakeAgent` is a conversation agent whose system
prompt explains the game.
"""
from __future__ import annotations

import re
from typing import Any, Dict, List, Optional, Tuple

import numpy as np

from ...rl.agentic.agents import model_agent
from ...rl.agentic.environments import base_environment

MOVES = {"up": (-1, 0), "down": (1, 0), "left": (0, -1), "right": (0, 1)}
SYSTEM_PROMPT = (
    "You are walking on a frozen lake. P is you, G is the goal, O is a hole, _ is safe ice. "
    "Each turn answer with exactly one move in the form ```Up```, ```Down```, ```Left``` or ```Right```. "
    "Reach G without stepping on O.")


def _solvable(board: np.ndarray) -> bool:
  n = board.shape[0]
  seen, stack = set(), [(0, 0)]
  while stack:
    r, c = stack.pop()
    if (r, c) in seen:
      continue
    seen.add((r, c))
    for dr, dc in MOVES.values():
      rr, cc = r + dr, c + dc
      if 0 <= rr < n and 0 <= cc < n and board[rr, cc] != "O":
        if board[rr, cc] == "G":
          return True
        stack.append((rr, cc))
  return False


def generate_map(size: int = 4, p_hole: float = 0.2, seed: int = 0) -> np.ndarray:
  """A size x size board with the start at the top-left; redrawn until a path to the goal exists."""
  rng = np.random.default_rng(seed)
  while True:
    board = np.where(rng.random((size, size)) < p_hole, "O", "_").astype("<U1")
    board[0, 0] = "_"
    gr, gc = divmod(int(rng.integers(1, size * size)), size)
    board[gr, gc] = "G"
    if _solvable(board):
      return board


def parse_move(text: str) -> Optional[str]:
  """The last fenced (or bare) move word of a reply."""
  found = re.findall(r"```\s*(up|down|left|right)\s*```", text, flags=re.I) or \
      re.findall(r"\b(up|down|left|right)\b", text, flags=re.I)
  return found[-1].lower() if found else None


class FrozenLakeEnv(base_environment.BaseTaskEnv):

  def __init__(self, task: Optional[Dict[str, Any]] = None, *, size: int = 4, p_hole: float = 0.2, seed: int = 0,
               max_steps: int = 8, **kwargs):
    task = task or {}
    super().__init__(task, max_steps=int(task.get("max_steps", max_steps)), **kwargs)
    self.size = int(task.get("size", size))
    self.p_hole = float(task.get("p_hole", p_hole))
    self.seed = int(task.get("seed", seed))
    self.board = generate_map(self.size, self.p_hole, self.seed)
    self.pos = (0, 0)

  def render(self) -> str:
    rows = []
    for r in range(self.size):
      rows.append(" ".join("P" if (r, c) == self.pos else str(self.board[r, c]) for c in range(self.size)))
    return "\n".join(rows)

  def _initial_observation(self) -> Dict[str, Any]:
    self.pos = (0, 0)
    return {"question": f"Current board:\n{self.render()}\nYour move?"}

  def _step_impl(self, action: Any) -> base_environment.EnvStepResult:
    move = parse_move(action if isinstance(action, str) else str(action))
    if move is None:
      return base_environment.EnvStepResult(
          {"question": f"Invalid answer. Reply with one move.\n{self.render()}"}, 0.0, False, {"valid": False})
    dr, dc = MOVES[move]
    r = min(max(self.pos[0] + dr, 0), self.size - 1)
    c = min(max(self.pos[1] + dc, 0), self.size - 1)
    self.pos = (r, c)
    cell = self.board[r, c]
    if cell == "G":
      return base_environment.EnvStepResult({"question": "You reached the goal."}, 1.0, True, {"valid": True})
    if cell == "O":
      return base_environment.EnvStepResult({"question": "You fell into a hole."}, 0.0, True, {"valid": True})
    return base_environment.EnvStepResult({"question": f"Current board:\n{self.render()}\nYour move?"}, 0.0, False,
                                          {"valid": True})

  @classmethod
  def from_dict(cls, env_args: Dict[str, Any]) -> "FrozenLakeEnv":
    env_args = dict(env_args)
    task = {k: env_args.pop(k) for k in ("size", "p_hole", "seed") if k in env_args}
    task.update(env_args.pop("task", None) or {})
    return cls(task, **env_args)


class FrozenLakeAgent(model_agent.ModelAgent):

  def __init__(self, system_prompt: str = SYSTEM_PROMPT, **kwargs):
    super().__init__(system_prompt=system_prompt, **kwargs)


def shortest_path_moves(env: FrozenLakeEnv) -> List[str]:
  """Breadth-first solution, used by tests and as an oracle policy."""
  from collections import deque
  start = (0, 0)
  prev: Dict[Tuple[int, int], Tuple[Tuple[int, int], str]] = {}
  q = deque([start])
  seen = {start}
  while q:
    cur = q.popleft()
    if env.board[cur] == "G":
      out = []
      while cur != start:
        cur, mv = prev[cur]
        out.append(mv)
      return out[::-1]
    for mv, (dr, dc) in MOVES.items():
      nxt = (cur[0] + dr, cur[1] + dc)
      if 0 <= nxt[0] < env.size and 0 <= nxt[1] < env.size and nxt not in seen and env.board[nxt] != "O":
        seen.add(nxt)
        prev[nxt] = (cur, mv)
        q.append(nxt)
  return []
