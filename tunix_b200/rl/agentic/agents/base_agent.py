"""Agent interfaces (tunix/rl/agentic/agents/base_agent.py:27-227)."""
from __future__ import annotations

import abc
import asyncio
import copy
from typing import Any, Dict, List, Optional

from . import agent_types


class LLMBaseAgent(abc.ABC):
  @property
  @abc.abstractmethod
  def chat_completions(self) -> List[Dict[str, str]]: ...

  @property
  @abc.abstractmethod
  def trajectory(self) -> agent_types.Trajectory: ...

  @abc.abstractmethod
  def update_from_env(self, observation: Any, reward: float, done: bool, info: Optional[Dict[str, Any]] = None,
                      **kwargs) -> None: ...

  @abc.abstractmethod
  def update_from_model(self, response: str, **kwargs) -> agent_types.Action: ...

  @abc.abstractmethod
  def reset(self) -> None: ...

  async def update_from_env_async(self, *args, **kwargs) -> None:
    return await asyncio.get_event_loop().run_in_executor(None, lambda: self.update_from_env(*args, **kwargs))

  async def update_from_model_async(self, *args, **kwargs) -> agent_types.Action:
    return await asyncio.get_event_loop().run_in_executor(None, lambda: self.update_from_model(*args, **kwargs))

  def get_current_step(self) -> Optional[agent_types.Step]:
    return self.trajectory.steps[-1] if self.trajectory.steps else None


class ConversationAgentBase(LLMBaseAgent):
  """Chat-style agent: keeps the message list sent to the model and the trajectory of steps."""

  def __init__(self, system_prompt: str):
    self.system_prompt = system_prompt
    self._trajectory = agent_types.Trajectory()
    self._messages: List[Dict[str, Any]] = []
    self._init_messages(system_prompt)
    self.step = 0

  def _init_messages(self, system_prompt: str) -> None:
    self._messages = [{"role": "system", "content": system_prompt or ""}]

  @staticmethod
  def _text(value: Any) -> str:
    """Dataset fields arrive as arrays of one element when a batch was split into examples."""
    if hasattr(value, "shape") and getattr(value, "size", 0) == 1:
      value = value.reshape(-1)[0]
      value = value.item() if hasattr(value, "item") else value
    if isinstance(value, (list, tuple)) and len(value) == 1:
      value = value[0]
    if isinstance(value, bytes):
      value = value.decode("utf-8", errors="replace")
    return "" if value is None else (value if isinstance(value, str) else str(value))

  def _observation_to_messages(self, observation: Any, reward: float, done: bool, info: Dict[str, Any]) -> None:
    if isinstance(observation, dict) and "prompts" in observation:
      self._messages.append({"role": "user", "content": self._text(observation["prompts"])})
    elif isinstance(observation, dict) and "question" in observation:
      self._messages.append({"role": "user", "content": self._text(observation["question"])})
    elif isinstance(observation, str):
      self._messages.append({"role": "user", "content": observation})

  @property
  def chat_completions(self) -> List[Dict[str, str]]:
    return self._messages

  @property
  def trajectory(self) -> agent_types.Trajectory:
    return self._trajectory

  def update_from_env(self, observation: Any, reward: float, done: bool, info: Optional[Dict[str, Any]] = None,
                      **kwargs) -> None:
    if self._trajectory.task is None:
      self._trajectory.task = {"prompts": [observation]} if isinstance(observation, str) else copy.deepcopy(observation)
    step = self.get_current_step()
    if step:
      step.observation, step.reward, step.done, step.info = observation, reward, done, info or {}
    if observation is not None:
      self._observation_to_messages(observation, reward, done, info or {})

  def reset(self) -> None:
    self._trajectory = agent_types.Trajectory()
    self._init_messages(self.system_prompt)
    self.step = 0
