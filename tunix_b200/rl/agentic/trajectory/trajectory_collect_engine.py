"""One agent-environment episode, asynchronously (tunix/rl/agentic/trajectory/trajectory_collect_engine.py:43-763).

reset -> repeat {model call -> agent.update_from_model -> env.step (bounded by the remaining
episode time) -> agent.update_from_env -> tokenise the turn} -> final reward -> Monte-Carlo
returns -> trajectory reward -> env.close (bounded).

Endings: the environment reports done (SUCCEEDED), `max_steps` turns (MAX_STEPS_REACHED), the
response-token budget is used up (MAX_CONTEXT_LIMIT_REACHED), the wall-clock budget is used up
(TIMEOUT), or `env.step` did not return in the time left (ENV_TIMEOUT). With `overlong_filter`
the token masks of episodes that ended in one of `filter_statuses` are zeroed, so they do not
train the policy, and their final reward is skipped.
"""
from __future__ import annotations

import asyncio
import inspect
import logging
import time
from typing import Any, AsyncGenerator, Callable, Dict, List, Optional, Set, Tuple

import numpy as np

from ..agents import agent_types
from ..agents.base_agent import ConversationAgentBase
from ..environments.base_environment import BaseTaskEnv
from .. import utils

_MODES = ("Trajectory", "Steps", "Token", "Conversation")
_CLOSE_TIMEOUT_S = 150.0
Status = agent_types.TrajectoryStatus


class _NoSpanTracer:
  class _Span:
    def __enter__(self): return self
    def __exit__(self, *a): return False

  def span(self, *a, **k):
    return self._Span()


class TrajectoryCollectEngine:
  def __init__(self, agent: ConversationAgentBase, env: BaseTaskEnv, *, model_call: Callable[..., Any],
               model_call_kwargs: Optional[Dict[str, Any]] = None, gamma: float = 1.0,
               max_response_length: Optional[int] = None, timeout: float = 600.0, tokenizer=None, chat_parser=None,
               filter_statuses: Optional[Set[Status]] = None, overlong_filter: bool = False, perf_v2=None):
    self.agent, self.env = agent, env
    self.model_call = model_call
    self.model_call_kwargs = model_call_kwargs or {}
    self.final_reward_fn = None
    self.max_steps = getattr(env, "max_steps", 1)
    self.gamma = gamma
    self.max_response_length = max_response_length
    self.timeout = timeout
    self.tokenizer, self.chat_parser = tokenizer, chat_parser
    self.filter_statuses = filter_statuses or {Status.MAX_STEPS_REACHED, Status.MAX_CONTEXT_LIMIT_REACHED,
                                               Status.TIMEOUT, Status.ENV_TIMEOUT}
    self.overlong_filter = overlong_filter
    self.perf_v2 = perf_v2 if perf_v2 is not None else _NoSpanTracer()
    self._response_token_count = 0
    self._start_ts = 0.0
    self._logged: Set[str] = set()
    self.env_time: Dict[str, Any] = {"reset_latency": 0.0, "step_latency": [], "close_latency": 0.0}
    self.reward_time: Dict[str, Any] = {"reward_latency": 0.0}
    if max_response_length is not None and not (tokenizer and chat_parser):
      logging.warning("max_response_length is set to %d, but no tokenizer or chat_parser is provided. response "
                      "length limits will not be enforced.", max_response_length)

  # ---- small helpers -------------------------------------------------------------------------
  @property
  def _debug_prefix(self) -> str:
    extra = getattr(self.env, "extra_kwargs", {}) or {}
    return (f"[step_idx={len(self.agent.trajectory.steps)}, pair_index={extra.get('pair_index')}, "
            f"group_id={extra.get('group_id')}]")

  async def _timed(self, fn: Callable[..., Any], *args, timeout: Optional[float] = None) -> Tuple[Any, float]:
    """Runs a blocking callable on the loop's executor; -> (result, wall seconds)."""
    t0 = time.perf_counter()
    fut = asyncio.get_running_loop().run_in_executor(None, fn, *args)
    res = await (asyncio.wait_for(fut, timeout=timeout) if timeout is not None else fut)
    return res, time.perf_counter() - t0

  def _clip(self, status: Status) -> None:
    self.agent.trajectory.status = status
    if status.name not in self._logged:
      self._logged.add(status.name)
      logging.warning("%s trajectory clipped: %s", self._debug_prefix, status.name)

  def _state_info(self, info: Optional[Dict[str, Any]]) -> Dict[str, Any]:
    out = dict(info or {})
    out["max_steps"] = self.max_steps
    out["cur_tokens"] = self._response_token_count
    return out

  def _budget_used_up(self) -> bool:
    if self.max_response_length is not None and self._response_token_count >= self.max_response_length:
      self._clip(Status.MAX_CONTEXT_LIMIT_REACHED)
      return True
    return False

  def _perf_tags(self) -> Dict[str, Any]:
    tags = {}
    extra = getattr(self.env, "extra_kwargs", None) or {}
    for key in ("group_id", "pair_index"):
      if extra.get(key) is not None:
        tags[key] = extra[key]
    pv = getattr(self.env, "task", {}).get("policy_version") if hasattr(self.env, "task") else None
    if pv is not None:
      tags["step"] = pv
    return tags

  # ---- episode phases ------------------------------------------------------------------------
  async def _reset(self) -> None:
    (obs, info), dt = await self._timed(self.env.reset)
    self.env_time["reset_latency"] += dt
    self.final_reward_fn = getattr(self.env, "final_reward_fn", None)
    self.agent.reset()
    self._start_ts = time.perf_counter()
    self._response_token_count = 0
    self.agent.update_from_env(observation=obs, reward=0.0, done=False, info=self._state_info(info))
    if self.tokenizer is not None and self.chat_parser is not None:
      toks, _ = utils.tokenize_and_generate_masks(self.agent.chat_completions, tokenizer=self.tokenizer,
                                                  parser=self.chat_parser, contains_first_msg=True,
                                                  contains_generation_msg=True)
      self.agent.trajectory.prompt_tokens = toks

  async def _call_model(self, max_generation_steps: Optional[int]):
    fn = self.model_call
    is_async = inspect.iscoroutinefunction(fn) or inspect.iscoroutinefunction(getattr(fn, "__call__", None))
    args = (self.agent.chat_completions, self.env)
    kw = dict(max_generation_steps=max_generation_steps, **self.model_call_kwargs)
    try:
      if is_async:
        return await fn(*args, **kw)
      return await asyncio.get_running_loop().run_in_executor(None, lambda: fn(*args, **kw))
    except Exception as e:
      logging.exception("Caught exception inside model_call: %s", e)
      raise

  def _record_tokens(self, step: agent_types.Step, out, done: bool, timed_out: bool) -> None:
    """Token-level record of the turn: the sampled tokens (mask 1) plus what the template appends
    after an assistant turn (mask 0), then the environment's messages (mask 0)."""
    assistant, env_msgs = utils.get_recent_assistant_user_messages(self.agent.chat_completions)
    if assistant:
      sampled = np.asarray(out.tokens[0])
      step.assistant_tokens, n_extra = self.chat_parser.update_assistant_end_tokens(sampled)
      step.assistant_masks = np.concatenate([np.ones(len(sampled), np.int32), np.zeros(n_extra, np.int32)])
      if step.logprobs is not None:
        step.logprobs = np.concatenate([np.asarray(step.logprobs, np.float32), np.zeros(n_extra, np.float32)])
    if env_msgs and not done and not timed_out:
      toks, masks = utils.tokenize_and_generate_masks(env_msgs, tokenizer=self.tokenizer, parser=self.chat_parser,
                                                      contains_first_msg=False, contains_generation_msg=True)
      step.env_tokens, step.env_masks = np.array(toks), np.array(masks)
      self._response_token_count += len(toks)

  async def _one_step(self) -> bool:
    if self._budget_used_up():
      return True
    budget = None if self.max_response_length is None else self.max_response_length - self._response_token_count
    out = await self._call_model(budget)
    if not self.agent.trajectory.steps and getattr(out, "left_padded_prompt_tokens", None) is not None:
      self.agent.trajectory.prompt_tokens = out.left_padded_prompt_tokens[0]
    if out.tokens is not None and len(out.tokens):
      self._response_token_count += len(out.tokens[0])
    action = self.agent.update_from_model(out.text[0]).action
    if action is None:
      logging.warning("Agent returned None action, using empty action list as fallback")
      action = []
    step_idx = len(self.agent.trajectory.steps)
    done = True
    if not self._budget_used_up():
      remaining = self.timeout - (time.perf_counter() - self._start_ts)
      try:
        with self.perf_v2.span("environment", tags=self._perf_tags()):
          (obs, rew, done, info), dt = await self._timed(self.env.step, action, timeout=max(remaining, 0.0))
      except asyncio.TimeoutError:
        self._clip(Status.ENV_TIMEOUT)
        logging.error("%s env.step hung at step %d and was abandoned after the %.1f s that were left.",
                      self._debug_prefix, step_idx, remaining)
        cur = self.agent.get_current_step()
        if cur is not None:
          cur.done = True
        return True
      self.env_time["step_latency"].append(dt)
      self.agent.update_from_env(obs, rew, done, self._state_info(info))
    cur = self.agent.get_current_step()
    if cur is not None and getattr(out, "logprobs", None) is not None:
      cur.logprobs = out.logprobs[0]
    timed_out = time.perf_counter() - self._start_ts > self.timeout
    if cur is not None and self.tokenizer and self.chat_parser:
      self._record_tokens(cur, out, done, timed_out)
    if timed_out:
      self._clip(Status.TIMEOUT)
      if cur is not None:
        cur.done = True
      return True
    return done

  async def _append_final_reward(self) -> None:
    last = self.agent.get_current_step()
    if last is None or not callable(self.final_reward_fn):
      return
    r, dt = await self._timed(self.final_reward_fn)
    self.reward_time["reward_latency"] += dt
    last.reward += r

  def compute_trajectory_reward(self):
    traj = self.agent.trajectory
    traj.reward = float(sum(s.reward for s in traj.steps))
    return traj

  def compute_mc_reward(self) -> None:
    g = 0.0
    for s in reversed(self.agent.trajectory.steps):
      g = s.reward + self.gamma * g
      s.mc_return = g

  async def _close(self) -> None:
    try:
      _, dt = await self._timed(self.env.close, timeout=_CLOSE_TIMEOUT_S)
      self.env_time["close_latency"] += dt
    except asyncio.TimeoutError:
      logging.error("%s env.close() did not return within %.0f s; its executor thread is leaked.",
                    self._debug_prefix, _CLOSE_TIMEOUT_S)

  # ---- public ----------------------------------------------------------------------------------
  async def collect(self, mode: str = "Conversation") -> Any:
    if mode not in _MODES:
      raise ValueError(f"Unsupported mode: {mode}, currently supported modes: {list(_MODES)}")
    await self._reset()
    traj = self.agent.trajectory
    traj.status = Status.RUNNING
    self._logged.clear()
    while True:
      if len(traj.steps) >= self.max_steps:
        self._clip(Status.MAX_STEPS_REACHED)
        break
      if await self._one_step():
        if traj.status == Status.RUNNING:
          traj.status = Status.SUCCEEDED
        break
    masked_out = self.overlong_filter and traj.status in self.filter_statuses
    try:
      if not masked_out:
        await self._append_final_reward()
      self.compute_mc_reward()
      self.compute_trajectory_reward()
    finally:
      await self._close()
    return self._render(mode, masked_out)

  def _render(self, mode: str, masked_out: bool) -> Any:
    traj = self.agent.trajectory
    if mode == "Trajectory":
      traj.env_time, traj.reward_time = self.env_time, self.reward_time
      return traj
    if mode == "Conversation":
      return self.agent.chat_completions
    if mode == "Steps":
      return [{"assistant_text": s.model_response, "env_text": s.observation, "done": s.done,
               "assistant_tokens": s.assistant_tokens if s.assistant_tokens is not None else [],
               "assistant_masks": s.assistant_masks if s.assistant_masks is not None else [],
               "env_tokens": s.env_tokens if s.env_tokens is not None else [],
               "env_masks": s.env_masks if s.env_masks is not None else [],
               "reward": s.reward, "mc_return": s.mc_return, "env_time": self.env_time,
               "reward_time": self.reward_time} for s in traj.steps]
    toks, masks, lps = [], [], []
    for s in traj.steps:
      if s.assistant_tokens is not None and len(s.assistant_tokens):
        toks.append(np.asarray(s.assistant_tokens))
        masks.append(np.asarray(s.assistant_masks))
        if s.logprobs is not None:
          assert len(s.logprobs) == len(s.assistant_tokens), (
              f"Logprobs length {len(s.logprobs)} does not match assistant tokens length {len(s.assistant_tokens)}")
          lps.append(np.asarray(s.logprobs))
        else:
          lps.append(np.zeros(len(s.assistant_tokens)))
      if s.env_tokens is not None and len(s.env_tokens):
        toks.append(np.asarray(s.env_tokens))
        masks.append(np.asarray(s.env_masks))
        lps.append(np.zeros(len(s.env_tokens)))
    cat = lambda xs: np.concatenate(xs, axis=0) if xs else np.array([], dtype=np.int32)
    conv_masks = cat(masks)
    extra = getattr(self.env, "extra_kwargs", {}) or {}
    return {"conversation_text": self.agent.chat_completions,
            "prompt_tokens": getattr(traj, "prompt_tokens", []),
            "conversation_tokens": cat(toks),
            "conversation_masks": np.zeros_like(conv_masks) if masked_out else conv_masks,
            "status": traj.status.name, "trajectory_reward": traj.reward, "env_time": self.env_time,
            "reward_time": self.reward_time, "old_logprobs": np.concatenate(lps, axis=0) if lps else None,
            "policy_version": getattr(self.env, "task", {}).get("policy_version"),
            "original_input": traj.task, "group_id": extra.get("group_id")}

  @staticmethod
  async def collect_multiple(pairs: List[Tuple[ConversationAgentBase, BaseTaskEnv]], *, model_call, gamma: float = 1.0,
                             timeout: float = 30.0, max_response_length: Optional[int] = None,
                             mode: str = "Trajectory", filter_statuses=None, overlong_filter: bool = True,
                             perf_v2=None, **engine_kwargs) -> AsyncGenerator[Tuple[int, Any], None]:
    """Runs the pairs concurrently and yields `(pair_index, result)` as episodes finish."""
    async def run(i, agent, env):
      eng = TrajectoryCollectEngine(agent, env, model_call=model_call, gamma=gamma, timeout=timeout,
                                    max_response_length=max_response_length, filter_statuses=filter_statuses,
                                    overlong_filter=overlong_filter, perf_v2=perf_v2, **engine_kwargs)
      return i, await eng.collect(mode=mode)
    for coro in asyncio.as_completed([run(i, a, e) for i, (a, e) in enumerate(pairs)]):
      yield await coro
