"""Agent interfaces (tunix/rl/agentic/agents/base_agent.py:27-227).

`LLMBaseAgent` is the contract the trajectory collector drives: the agent owns the conversation sent to the model
(`chat_completions`) and the record of the episode (`trajectory`); the collector alternates `update_from_env`
(observation, reward, done, info) and `update_from_model` (raw response -> `Action`). The async variants run the
blocking methods off the event loop.

`ConversationAgentBase` implements the bookkeeping every chat-style agent shares: a message list that starts with
the system prompt, the task recorded from the first observation, the last step completed with what the environment
answered, and a small *observation reader* table - which keys of a dict observation carry the next user turn -
that subclasses extend instead of re-writing the whole method.
"""
from __future__ import annotations

import abc
import asyncio
import copy
from typing import Any, Callable, Dict, List, Optional, Sequence

from . import agent_types

Message = Dict[str, Any]


def scalar_text(value: Any) -> str:
  """A dataset field as text. Batches split into examples leave one-element arrays, lists and byte strings."""
  if getattr(value, "size", None) == 1 and hasattr(value, "reshape"):
    value = value.reshape(-1)[0]
    value = value.item() if hasattr(value, "item") else value
  if isinstance(value, (list, tuple)) and len(value) == 1:
    value = value[0]
  if isinstance(value, bytes):
    return value.decode("utf-8", errors="replace")
  if value is None:
    return ""
  return value if isinstance(value, str) else str(value)


class LLMBaseAgent(abc.ABC):

  @property
  @abc.abstractmethod
  def chat_completions(self) -> List[Dict[str, str]]:
    """The messages to send to the model next."""

  @property
  @abc.abstractmethod
  def trajectory(self) -> agent_types.Trajectory:
    """The episode so far."""

  @abc.abstractmethod
  def update_from_env(self, observation: Any, reward: float, done: bool, info: Optional[Dict[str, Any]] = None,
                      **kwargs) -> None:
    """Takes in what the environment returned for the last action (or the first observation)."""

  @abc.abstractmethod
  def update_from_model(self, response: str, **kwargs) -> agent_types.Action:
    """Takes in the model's raw response and returns the action to apply."""

  @abc.abstractmethod
  def reset(self) -> None:
    """Starts a new episode."""

  async def update_from_env_async(self, *args, **kwargs) -> None:
    await asyncio.to_thread(self.update_from_env, *args, **kwargs)

  async def update_from_model_async(self, *args, **kwargs) -> agent_types.Action:
    return await asyncio.to_thread(self.update_from_model, *args, **kwargs)

  def get_current_step(self) -> Optional[agent_types.Step]:
    steps = self.trajectory.steps
    return steps[-1] if steps else None


class ConversationAgentBase(LLMBaseAgent):
  user_turn_keys: Sequence[str] = ("prompts", "question")     # keys of a dict observation that hold the next user turn

  def __init__(self, system_prompt: str):
    self.system_prompt = system_prompt
    self.reset()

  # ---- conversation
  def _init_messages(self, system_prompt: str) -> None:
    self._messages: List[Message] = [{"role": "system", "content": system_prompt or ""}]

  _text = staticmethod(scalar_text)

  def _user_turn_of(self, observation: Any) -> Optional[str]:
    if isinstance(observation, str):
      return observation
    if isinstance(observation, dict):
      for key in self.user_turn_keys:
        if key in observation:
          return scalar_text(observation[key])
    return None

  def _observation_to_messages(self, observation: Any, reward: float, done: bool, info: Dict[str, Any]) -> None:
    turn = self._user_turn_of(observation)
    if turn is not None:
      self._messages.append({"role": "user", "content": turn})

  @property
  def chat_completions(self) -> List[Dict[str, str]]:
    return self._messages

  # ---- episode record
  @property
  def trajectory(self) -> agent_types.Trajectory:
    return self._trajectory

  def update_from_env(self, observation: Any, reward: float, done: bool, info: Optional[Dict[str, Any]] = None,
                      **kwargs) -> None:
    info = info or {}
    if self._trajectory.task is None:              # the first observation is the task
      self._trajectory.task = {"prompts": [observation]} if isinstance(observation, str) else copy.deepcopy(observation)
    last = self.get_current_step()
    if last is not None:                            # what the environment answered belongs to the step that acted
      last.observation, last.reward, last.done, last.info = observation, reward, done, info
    if observation is not None:
      self._observation_to_messages(observation, reward, done, info)

  def reset(self) -> None:
    self._trajectory = agent_types.Trajectory()
    self._init_messages(self.system_prompt)
    self.step = 0
