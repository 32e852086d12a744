"""Stand-ins for the expensive parts of an RL job, for tests and demos of the control plane
(tunix/experimental/common/test_utils.py:35-440): an environment with a scripted episode, a pool of them, a
character-level tokenizer, a chat parser, a sampler service that answers without a model, an agent, a trainer and a
small orchestrator that drives them through collect -> train -> sync.

Everything is deterministic: replies, rewards and token ids are pure functions of the inputs, so two runs of a test
produce the same trajectories. `gpu_only` plays the role of the reference's accelerator-only decorator."""
from __future__ import annotations

import asyncio
import functools
import threading
import time
import zlib
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

from ...rl.agentic.agents import agent_types, base_agent
from ...rl.agentic.environments import base_environment
from ..rollout import sampler as sampler_lib


def _digest(text: str) -> int:
  return zlib.crc32(text.encode("utf-8"))


class MockEnvironment(base_environment.BaseTaskEnv):
  """An episode of `turns` steps. Every step costs `delay_seconds` of wall time (an environment is slow, that is
  why rollouts are asynchronous); the reward of a step is 1.0 when the action mentions the step's keyword."""

  def __init__(self, env_id: str = "mock_env_01", delay_seconds: float = 0.05, turns: int = 2,
               keywords: Sequence[str] = ("alpha", "beta", "gamma"), **kwargs):
    super().__init__(task={"env_id": env_id}, max_steps=turns, **kwargs)
    self.env_id, self.delay_seconds, self.keywords = env_id, float(delay_seconds), tuple(keywords)
    self.closed = False
    self.history: List[str] = []

  def _keyword(self) -> str:
    return self.keywords[self.step_count % len(self.keywords)]

  def _initial_observation(self) -> Dict[str, Any]:
    self.history.clear()
    return {"question": f"[{self.env_id}] say {self._keyword()}"}

  def _step_impl(self, action: Any) -> base_environment.EnvStepResult:
    if self.delay_seconds:
      time.sleep(self.delay_seconds)
    said = str(getattr(action, "action", action))
    wanted = self.keywords[(self.step_count - 1) % len(self.keywords)]
    self.history.append(said)
    reward = 1.0 if wanted in said else 0.0
    if self.step_count >= self.max_steps:
      return base_environment.EnvStepResult(observation={}, reward=reward, done=True, info={"response": said})
    return self.turn({"question": f"[{self.env_id}] now say {self._keyword()}"}, response=said, reward=reward)

  def close(self) -> None:
    self.closed = True


class MockEnvironmentPool:
  """A fixed number of environments handed out under a lock; `acquire_env` blocks (up to `timeout`) while all are
  out."""

  def __init__(self, size: int = 2, env_factory: Optional[Callable[[int], MockEnvironment]] = None):
    make = env_factory or (lambda i: MockEnvironment(env_id=f"mock_env_{i:02d}", delay_seconds=0.0))
    self._free: List[MockEnvironment] = [make(i) for i in range(size)]
    self._out: set = set()
    self._cv = threading.Condition()
    self.size = size

  def acquire_env(self, timeout: Optional[float] = None) -> MockEnvironment:
    with self._cv:
      if not self._cv.wait_for(lambda: bool(self._free), timeout):
        raise TimeoutError(f"no environment free after {timeout} s ({len(self._out)} out)")
      env = self._free.pop()
      self._out.add(id(env))
      return env

  def release_env(self, env: MockEnvironment) -> None:
    with self._cv:
      if id(env) not in self._out:
        raise ValueError("environment does not belong to this pool or was released twice")
      self._out.discard(id(env))
      self._free.append(env)
      self._cv.notify()

  @property
  def available(self) -> int:
    with self._cv:
      return len(self._free)


class MockTokenizer:
  """One id per character (code point + 3; 0 pad, 1 bos, 2 eos), so `decode(encode(s)) == s`."""

  PAD, BOS, EOS, SHIFT = 0, 1, 2, 3

  def encode(self, text: str, add_special_tokens: bool = False) -> List[int]:
    body = [ord(c) + self.SHIFT for c in text]
    return [self.BOS] + body if add_special_tokens else body

  def decode(self, ids: Sequence[int], **kwargs) -> str:
    return "".join(chr(int(i) - self.SHIFT) for i in ids if int(i) >= self.SHIFT)

  def dedup_bos_ids(self, tokens: List[int]) -> List[int]:
    start = 0
    while start + 1 < len(tokens) and tokens[start] == self.BOS and tokens[start + 1] == self.BOS:
      start += 1
    return list(tokens[start:])

  def pad_id(self) -> int:
    return self.PAD

  def bos_id(self) -> int:
    return self.BOS

  def eos_id(self) -> int:
    return self.EOS


class MockChatParser:
  """`<role>content</role>` per message; the generation prompt is an open `<assistant>`."""

  assistant_token = "<assistant>"

  def __init__(self):
    self.end_tokens: Tuple[str, ...] = ("</assistant>",)

  def parse(self, messages: Sequence[Dict[str, str]], add_generation_prompt: bool = False,
            is_first_msg: bool = False) -> str:
    text = "".join(f"<{m['role']}>{m.get('content') or ''}</{m['role']}>" for m in messages)
    return text + (self.assistant_token if add_generation_prompt else "")

  def update_assistant_end_tokens(self, end_tokens: Sequence[str]) -> None:
    self.end_tokens = tuple(end_tokens)


class MockSampler:
  """A sampler service without a model (the `experimental.rollout.sampler.Sampler` protocol): the reply to a prompt
  is `reply_fn(prompt text, policy version)`, tokenised with `MockTokenizer`; log-probs are a fixed -0.5. Counts
  what a test wants to assert on: requests served, weight-sync phases seen, KV migrations."""

  def __init__(self, reply_fn: Optional[Callable[[str, int], str]] = None, latency_s: float = 0.0,
               tokenizer: Optional[MockTokenizer] = None):
    self.tokenizer = tokenizer or MockTokenizer()
    self._reply = reply_fn or (lambda prompt, version: f"alpha beta gamma v{version}")
    self.latency_s = float(latency_s)
    self.policy_version = 0
    self.served = 0
    self.phases: List[str] = []
    self.migrations: List[Any] = []
    self._paused = asyncio.Event()
    self._running = 0

  def initialize(self) -> None:
    self._paused.clear()

  async def start(self, **kwargs) -> None:
    self.initialize()

  async def stop(self, **kwargs) -> None:
    self.phases.append("stop")

  async def pause(self, **kwargs) -> None:
    self._paused.set()

  async def resume(self, **kwargs) -> None:
    self._paused.clear()

  async def get_mesh(self, **kwargs) -> Any:
    return None

  def _prompt_text(self, prompt: Any) -> str:
    if isinstance(prompt, str):
      return prompt
    if isinstance(prompt, (list, tuple)) and prompt and isinstance(prompt[0], dict):
      return MockChatParser().parse(prompt, add_generation_prompt=True)
    return self.tokenizer.decode(np.asarray(prompt).reshape(-1).tolist())

  async def sample(self, sampling_requests: Sequence[Any], **kwargs) -> List[sampler_lib.SamplingResponse]:
    if self._paused.is_set():
      return [sampler_lib.SamplingResponse(finish_reason="cancelled") for _ in sampling_requests]
    self._running += len(sampling_requests)
    try:
      if self.latency_s:
        await asyncio.sleep(self.latency_s)
      out = []
      for req in sampling_requests:
        prompt = self._prompt_text(getattr(req, "prompt", req))
        params = getattr(req, "sampling_params", None) or sampler_lib.SamplingParams()
        ids = self.tokenizer.encode(self._reply(prompt, self.policy_version))
        cut = ids[:params.max_tokens]
        out.append(sampler_lib.SamplingResponse(
            text=self.tokenizer.decode(cut), prompt_token_ids=np.asarray(self.tokenizer.encode(prompt), np.int32),
            token_ids=np.asarray(cut, np.int32),
            logprobs=np.full(len(cut), -0.5, np.float32) if params.return_logprobs else None,
            finish_reason="length" if len(cut) < len(ids) else "stop"))
        self.served += 1
      return out
    finally:
      self._running -= len(sampling_requests)

  async def bind_weight_sync(self, **kwargs) -> None:
    self.phases.append("bind")

  async def get_weight_sync_metadata(self, **kwargs) -> List[Any]:
    return []

  async def pre_weight_sync(self, sync_request: Any = None, **kwargs) -> None:
    self.phases.append("pre")

  async def weight_sync(self, sync_request: Any = None, **kwargs) -> None:
    self.phases.append("transfer")

  async def post_weight_sync(self, sync_request: Any = None, **kwargs) -> None:
    self.phases.append("post")
    version = getattr(sync_request, "policy_version", None)
    self.policy_version = self.policy_version + 1 if version is None else int(version)

  async def abort_weight_sync(self, sync_request: Any = None, **kwargs) -> None:
    self.phases.append("abort")

  async def get_weight_sync_status(self, **kwargs) -> Dict[str, Any]:
    return {"policy_version": self.policy_version, "phases": list(self.phases)}

  async def migrate_kv_cache(self, target: Any = None, **kwargs) -> None:
    self.migrations.append(target)

  async def get_load_info(self, **kwargs) -> sampler_lib.LoadInfo:
    return sampler_lib.LoadInfo(num_requests_running=self._running)


MockBaseSamplerImpl = MockSampler      # the reference's name for the same role


class MockAgent(base_agent.ConversationAgentBase):
  """Turns the model's text into an action unchanged and records the step."""

  def __init__(self, system_prompt: str = "Mock Agent"):
    super().__init__(system_prompt)

  def update_from_model(self, response: str, **kwargs) -> agent_types.Action:
    self._messages.append({"role": "assistant", "content": response})
    step = agent_types.Step(model_response=response, action=agent_types.Action(action=response))
    self._trajectory.steps.append(step)
    return step.action


class MockTrainer:
  """Counts steps; a "weight" is the running mean reward it has seen, which makes training observable."""

  def __init__(self, trainer_id: str = "trainer_01"):
    self.trainer_id = trainer_id
    self.train_steps = 0
    self.policy_version = 0
    self.mean_reward = 0.0
    self.pushed_to: List[str] = []

  def train_step(self, batch: Any) -> int:
    rewards = [float(getattr(item, "reward", 0.0)) for item in (batch or [])]
    if rewards:
      self.mean_reward += (sum(rewards) / len(rewards) - self.mean_reward) / (self.train_steps + 1)
    self.train_steps += 1
    return self.train_steps

  def push_weights(self, peer_addresses: Optional[List[str]] = None) -> int:
    self.policy_version += 1
    self.pushed_to.extend(peer_addresses or [])
    return self.policy_version


class _Episode:
  """What one rollout produced: the conversation's reward and how many steps it took."""

  def __init__(self, env_id: str, reward: float, steps: int, policy_version: int):
    self.env_id, self.reward, self.steps, self.policy_version = env_id, reward, steps, policy_version


class MockGlobalOrchestrator:
  """collect (episodes run concurrently, bounded by the pool) -> train -> sync, with all parts in this process."""

  def __init__(self, num_envs: int = 2, sampler: Optional[MockSampler] = None, trainer: Optional[MockTrainer] = None,
               pool: Optional[MockEnvironmentPool] = None):
    self.pool = pool or MockEnvironmentPool(num_envs)
    self.sampler = sampler or MockSampler()
    self.trainer = trainer or MockTrainer()
    self.running = False

  def start_workers(self) -> None:
    self.sampler.initialize()
    self.running = True

  def stop_workers(self) -> None:
    self.running = False

  async def _episode(self) -> _Episode:
    loop = asyncio.get_running_loop()
    env = await loop.run_in_executor(None, self.pool.acquire_env, 30.0)
    try:
      agent = MockAgent()
      observation, _ = env.reset()
      agent.update_from_env(observation, 0.0, False, {})
      total, steps, done = 0.0, 0, False
      while not done:
        request = sampler_lib.SamplingRequest(prompt=agent.chat_completions)
        reply = (await self.sampler.sample([request]))[0]
        action = agent.update_from_model(reply.text)
        observation, reward, done, info = await loop.run_in_executor(None, env.step, action)
        agent.update_from_env(observation, reward, done, info)
        total, steps = total + reward, steps + 1
      return _Episode(env.env_id, total, steps, self.sampler.policy_version)
    finally:
      self.pool.release_env(env)

  async def collect_rollout_batch(self, batch_size: int) -> List[_Episode]:
    if not self.running:
      raise RuntimeError("start_workers() first")
    return list(await asyncio.gather(*(self._episode() for _ in range(batch_size))))

  async def run_training_step(self, batch: Sequence[_Episode]) -> int:
    return await asyncio.get_running_loop().run_in_executor(None, self.trainer.train_step, list(batch))

  def synchronize_weights(self, peer_addresses: Optional[List[str]] = None) -> int:
    version = self.trainer.push_weights(peer_addresses)
    request = type("SyncRequest", (), {"policy_version": version})()
    async def rounds():
      for phase in (self.sampler.pre_weight_sync, self.sampler.weight_sync, self.sampler.post_weight_sync):
        await phase(request)
    try:
      asyncio.get_running_loop()
    except RuntimeError:
      asyncio.run(rounds())
    else:
      raise RuntimeError("synchronize_weights() is synchronous: call it outside the event loop")
    return version


def is_gpu_available() -> bool:
  try:
    import torch
    return bool(torch.cuda.is_available())
  except Exception:  # noqa: BLE001
    return False


def gpu_only(func: Callable[..., Any]) -> Callable[..., Any]:
  """Skips a test (unittest.SkipTest, which pytest honours too) on a machine without a GPU."""
  @functools.wraps(func)
  def wrapper(*args, **kwargs):
    if not is_gpu_available():
      import unittest
      raise unittest.SkipTest("needs a GPU")
    return func(*args, **kwargs)
  return wrapper
