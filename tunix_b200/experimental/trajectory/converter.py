"""Between the agent stack's episode record and the stored trajectory schema
(tunix/experimental/trajectory/converter.py:28-426).

An episode is a list of *turns* (`agent_types.Step`: model response, parsed action, the environment's answer,
token-level record). A stored trajectory is a flat list of *steps* with a source each. The mapping is positional:

    stored step 0          the task prompt                         (source USER)
    stored step 2 t + 1    the agent half of turn t                (source AGENT:  response, thought, tool calls,
                                                                    sampled tokens / masks / log-probs, return)
    stored step 2 t + 2    the environment half of turn t          (source SYSTEM: observation, reward, done,
                                                                    environment tokens / masks)

`EpisodeWriter` goes one way (turns -> steps, also turn by turn while an episode is still running),
`to_tunix_trajectory` goes back, tolerating records in which an agent step has no environment step after it or
environment steps stand alone. The raw action is kept under `extra["raw_action"]` so that the round trip does not
depend on how well `action_converter` understood it.
"""
from __future__ import annotations

from typing import Any, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple, Union

import numpy as np

from ...rl.agentic.agents import agent_types
from . import action_converter
from . import trajectory as trajectory_lib

_ACTION_KEYS = ("raw_action", "action")       # where a stored agent step may keep the original action


def agent_step_id(turn: int) -> int:
  return 2 * turn + 1


def env_step_id(turn: int) -> int:
  return 2 * turn + 2


# ------------------------------------------------------------------------------------ episode -> stored steps
def _token_metrics(tokens: Any, logprobs: Any) -> Optional[trajectory_lib.Metrics]:
  """Completion length, ids and log-probs as schema metrics (None when the turn has neither)."""
  ids = [int(t) for t in tokens] if isinstance(tokens, (list, tuple, np.ndarray)) else None
  lps = [float(x) for x in logprobs] if isinstance(logprobs, (list, tuple, np.ndarray)) else None
  if ids is None and lps is None:
    return None
  if ids is not None and lps is not None and len(ids) != len(lps):
    raise ValueError(f"Length of assistant_tokens ({len(ids)}) must match length of logprobs ({len(lps)}).")
  return trajectory_lib.Metrics(completion_tokens=None if ids is None else len(ids), completion_token_ids=ids, logprobs=lps)


def _observation_record(observation: Any) -> Optional[trajectory_lib.Observation]:
  if observation is None:
    return None
  parts = observation if isinstance(observation, list) else [observation]
  return trajectory_lib.Observation(results=[trajectory_lib.ObservationResult(content=str(p)) for p in parts])


def _task_text(task: Any) -> Optional[str]:
  if isinstance(task, str):
    return task or None
  if isinstance(task, dict):
    prompts = task.get("prompts")
    if isinstance(prompts, str):
      return prompts or None
    if isinstance(prompts, list) and prompts:
      return str(prompts[0]) or None
  return None


def create_task_step(task: Any) -> Optional[trajectory_lib.TunixEnvStep]:
  """Stored step 0 from a task (a prompt string or a dict with `prompts`); None when there is no prompt."""
  text = _task_text(task)
  if text is None:
    return None
  return trajectory_lib.TunixEnvStep(step_id=0, source=trajectory_lib.Source.USER, message=text)


def create_agent_step(step: Optional[agent_types.Step], tunix_step_id: int) -> Optional[trajectory_lib.TunixAgentStep]:
  """The agent half of turn `tunix_step_id` (stored id 2 t + 1)."""
  if step is None:
    return None
  extra = dict(step.info or {})
  raw = step.action.action if isinstance(step.action, agent_types.Action) else step.action
  if raw is not None:
    extra["raw_action"] = raw
  return trajectory_lib.TunixAgentStep(
      step_id=agent_step_id(tunix_step_id), source=trajectory_lib.Source.AGENT, message=step.model_response,
      reasoning_content=step.thought or None, tool_calls=action_converter.extract_tool_calls(step.action),
      metrics=_token_metrics(step.assistant_tokens, step.logprobs), assistant_tokens=step.assistant_tokens,
      assistant_masks=step.assistant_masks, logprobs=step.logprobs, mc_return=step.mc_return or None,
      extra=extra or None)


def create_env_step(step: Optional[agent_types.Step], tunix_step_id: int) -> Optional[trajectory_lib.TunixEnvStep]:
  """The environment half of turn `tunix_step_id` (stored id 2 t + 2)."""
  if step is None:
    return None
  return trajectory_lib.TunixEnvStep(
      step_id=env_step_id(tunix_step_id), source=trajectory_lib.Source.SYSTEM,
      message="" if step.observation is None else str(step.observation),
      observation=_observation_record(step.observation), reward=step.reward, done=step.done,
      env_tokens=step.env_tokens, env_masks=step.env_masks, extra=step.info or None)


class EpisodeWriter:
  """Turns -> stored steps, incrementally: `task()` once, then `turn()` for every finished turn. Used by
  collectors that append to a trajectory store while the episode is still running."""

  def __init__(self) -> None:
    self.turns = 0

  def task(self, task: Any) -> List[trajectory_lib.TunixEnvStep]:
    first = create_task_step(task)
    return [] if first is None else [first]

  def turn(self, step: agent_types.Step) -> List[Union[trajectory_lib.TunixAgentStep, trajectory_lib.TunixEnvStep]]:
    pair = [create_agent_step(step, self.turns), create_env_step(step, self.turns)]
    self.turns += 1
    return pair

  def episode(self, traj: agent_types.Trajectory) -> List[Any]:
    """All stored steps of a finished episode. Without a task prompt the ids would start at 1, which the schema
    does not allow, so an empty task step stands in."""
    head = self.task(traj.task) or [trajectory_lib.TunixEnvStep(step_id=0, source=trajectory_lib.Source.USER, message="")]
    return head + [s for step in traj.steps for s in self.turn(step)]


def from_tunix_trajectory(traj: agent_types.Trajectory, traj_id: str, request: Any = None, agent: Any = None,
                          target_policy_versions: Optional[List[int]] = None) -> trajectory_lib.TunixTrajectory:
  """A whole finished episode as a stored trajectory (metadata from `create_trajectory_metadata`)."""
  md = create_trajectory_metadata(traj_id, request=request, agent=agent, target_policy_versions=target_policy_versions,
                                  status=traj.status.name)
  fields = md.model_dump()
  fields.update(total_reward=float(traj.reward), env_time=traj.env_time or None, reward_time=traj.reward_time or None)
  return trajectory_lib.TunixTrajectory(**fields, steps=EpisodeWriter().episode(traj))


# ------------------------------------------------------------------------------------ stored steps -> episode
def _array(values: Any) -> Optional[np.ndarray]:
  return None if values is None else np.asarray(values)


def _without_action(extra: Optional[Dict[str, Any]]) -> Dict[str, Any]:
  return {k: v for k, v in (extra or {}).items() if k not in _ACTION_KEYS}


def _stored_action(agent_step: trajectory_lib.TunixAgentStep) -> Optional[agent_types.Action]:
  """The original action if it was kept, else one rebuilt from the tool calls (a single call is unwrapped)."""
  extra = agent_step.extra or {}
  for key in _ACTION_KEYS:
    if key in extra:
      return agent_types.Action(action=extra[key])
  if not agent_step.tool_calls:
    return None
  calls = [{"id": c.tool_call_id, "name": c.function_name, "arguments": c.arguments} for c in agent_step.tool_calls]
  return agent_types.Action(action=calls[0] if len(calls) == 1 else calls)


def _agent_half(agent_step: trajectory_lib.TunixAgentStep) -> Dict[str, Any]:
  metrics = agent_step.metrics
  tokens, logprobs = agent_step.assistant_tokens, agent_step.logprobs
  if metrics is not None:                      # the schema's own metrics can stand in for the token arrays
    if tokens is None and metrics.completion_token_ids is not None:
      tokens = metrics.completion_token_ids
    if logprobs is None and metrics.logprobs is not None:
      logprobs = metrics.logprobs
  return dict(model_response=agent_step.message or "", thought=agent_step.reasoning_content or "",
              action=_stored_action(agent_step), assistant_tokens=_array(tokens),
              assistant_masks=_array(agent_step.assistant_masks), logprobs=_array(logprobs),
              mc_return=0.0 if agent_step.mc_return is None else float(agent_step.mc_return))


def _env_half(env_step: trajectory_lib.TunixEnvStep) -> Dict[str, Any]:
  results = env_step.observation.results if env_step.observation is not None else []
  if results:
    observation: Any = results[0].content if len(results) == 1 else [r.content for r in results]
  else:
    observation = env_step.message or None
  return dict(observation=observation, reward=0.0 if env_step.reward is None else float(env_step.reward),
              done=bool(env_step.done), env_tokens=_array(env_step.env_tokens), env_masks=_array(env_step.env_masks))


def to_tunix_step(agent_step: Optional[trajectory_lib.TunixAgentStep] = None,
                  env_step: Optional[trajectory_lib.TunixEnvStep] = None) -> agent_types.Step:
  """One turn from its stored halves (either may be missing; both missing gives an empty turn)."""
  fields: Dict[str, Any] = {}
  info: Dict[str, Any] = {}
  for half, read in ((agent_step, _agent_half), (env_step, _env_half)):
    if half is not None:
      fields.update(read(half))
      info.update(_without_action(half.extra))
  return agent_types.Step(info=info, **fields)


def _turns(steps: Sequence[Any]) -> Iterator[Tuple[Optional[Any], Optional[Any]]]:
  """Pairs stored steps into (agent half, environment half): an agent step takes the step after it unless that is
  another agent step; an environment step with no agent step before it forms a turn of its own."""
  i = 0
  while i < len(steps):
    here = steps[i]
    if here.source != trajectory_lib.Source.AGENT:
      yield None, here
      i += 1
      continue
    after = steps[i + 1] if i + 1 < len(steps) and steps[i + 1].source != trajectory_lib.Source.AGENT else None
    yield here, after
    i += 1 if after is None else 2


def to_tunix_trajectory(traj: Union[trajectory_lib.TunixTrajectory, Dict[str, Any]]) -> agent_types.Trajectory:
  """An episode record from a stored trajectory (or its JSON dict)."""
  stored = trajectory_lib.TunixTrajectory.from_json_dict(traj) if isinstance(traj, dict) else traj
  steps = list(stored.steps)
  task = None
  if steps and steps[0].source in (trajectory_lib.Source.USER, trajectory_lib.Source.SYSTEM):
    task = {"prompts": [steps[0].message]}
    steps = steps[1:]
  status = getattr(agent_types.TrajectoryStatus, str(stored.status), None) if stored.status is not None else None
  return agent_types.Trajectory(
      task=task, steps=[to_tunix_step(agent_step=a, env_step=e) for a, e in _turns(steps)],
      reward=0.0 if stored.total_reward is None else float(stored.total_reward),
      status=status if isinstance(status, agent_types.TrajectoryStatus) else agent_types.TrajectoryStatus.RUNNING,
      env_time=stored.env_time or {}, reward_time=getattr(stored, "reward_time", None) or {})


# ------------------------------------------------------------------------------------ metadata
def create_trajectory_metadata(traj_id: str, request: Any = None, agent: Any = None,
                               target_policy_versions: Optional[List[int]] = None, status: str = "RUNNING",
                               extra: Optional[Dict[str, Any]] = None) -> trajectory_lib.TunixTrajectoryMetadata:
  """Metadata of a stored trajectory from the rollout request that caused it and the agent that produced it."""
  record = agent if isinstance(agent, trajectory_lib.Agent) else trajectory_lib.Agent(
      name=getattr(agent, "name", "agent"), version=getattr(agent, "version", "1.0"))
  episode = getattr(agent, "trajectory", None)
  merged = {**(getattr(request, "metadata", None) or {}), **(extra or {})}
  return trajectory_lib.TunixTrajectoryMetadata(
      trajectory_id=traj_id, agent=record, prompt_id=getattr(request, "prompt_id", None),
      group_offset_id=getattr(request, "group_offset_id", None), target_policy_versions=target_policy_versions,
      status=status, total_reward=getattr(episode, "reward", None),
      hyperparams=getattr(request, "generation_kwargs", None), env_time=getattr(episode, "env_time", None),
      reward_time=getattr(episode, "reward_time", None), extra=merged or None)
