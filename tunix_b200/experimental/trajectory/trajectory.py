"""Agent trajectory records: the ATIF interchange schema plus token-level RL fields.

The base models follow the public Agent Trajectory Interchange Format (schema
version ATIF-v1.7): a trajectory is metadata (agent, session, final metrics)
plus an ordered list of steps, each step from the system, the user or the agent.
The ``Tunix*`` models add what an RL learner needs per step (token ids, loss
masks, sampling log-probs, the policy version that produced them, rewards).

Behaviour matches tunix/experimental/trajectory/trajectory.py (field names,
validators, 1-based step ids for ATIF and 0-based for the RL variant), so a
file written by one side loads on the other.
"""

from __future__ import annotations

import datetime
import enum
from typing import Annotated, Any

import numpy as np
import pydantic

SCHEMA_VERSION = "ATIF-v1.7"

MetadataDict = dict[str, Any] | None


def _to_int_array(v):
  if v is None:
    return None
  return np.asarray(v, dtype=np.int32)


def _to_float_array(v):
  if v is None:
    return None
  return np.asarray(v, dtype=np.float32)


def _array_to_list(v):
  return None if v is None else np.asarray(v).tolist()


IntArray = Annotated[
    Any,
    pydantic.BeforeValidator(_to_int_array),
    pydantic.PlainSerializer(_array_to_list, return_type=list | None),
]
FloatArray = Annotated[
    Any,
    pydantic.BeforeValidator(_to_float_array),
    pydantic.PlainSerializer(_array_to_list, return_type=list | None),
]


class TrajectoryError(ValueError):
  """A trajectory that breaks the schema's structural rules."""


class Source(str, enum.Enum):
  SYSTEM = "system"
  USER = "user"
  AGENT = "agent"


class _Strict(pydantic.BaseModel):
  model_config = pydantic.ConfigDict(extra="forbid")


class ToolCall(_Strict):
  tool_call_id: str
  function_name: str
  arguments: dict[str, Any] = pydantic.Field(default_factory=dict)
  extra: MetadataDict = None


class SubagentTrajectoryRef(_Strict):
  """Pointer from an observation to a sub-agent's trajectory."""

  trajectory_id: str | None = None
  session_id: str | None = None
  trajectory_path: str | None = None
  extra: MetadataDict = None

  @pydantic.model_validator(mode="after")
  def _needs_target(self):
    if not (self.trajectory_id or self.session_id or self.trajectory_path):
      raise ValueError(
          "a subagent reference needs trajectory_id, session_id or trajectory_path")
    return self


class ObservationResult(_Strict):
  source_call_id: str | None = None
  content: Any = None
  subagent_trajectory_ref: list[SubagentTrajectoryRef] | None = None
  extra: MetadataDict = None


class Observation(_Strict):
  results: list[ObservationResult] = pydantic.Field(default_factory=list)


class Metrics(_Strict):
  prompt_tokens: int | None = None
  completion_tokens: int | None = None
  cached_tokens: int | None = None
  cost_usd: float | None = None
  prompt_token_ids: list[int] | None = None
  completion_token_ids: list[int] | None = None
  logprobs: list[float] | None = None
  extra: MetadataDict = None


class FinalMetrics(_Strict):
  total_prompt_tokens: int | None = None
  total_completion_tokens: int | None = None
  total_cached_tokens: int | None = None
  total_cost_usd: float | None = None
  total_steps: int | None = None
  extra: MetadataDict = None


_AGENT_ONLY = ("model_name", "reasoning_effort", "reasoning_content",
               "tool_calls", "metrics")


class Step(_Strict):
  """One turn. Agent-only fields are rejected on system and user steps."""

  step_id: int = pydantic.Field(ge=0)
  timestamp: datetime.datetime | None = None
  source: Source
  model_name: str | None = None
  reasoning_effort: str | float | None = None
  message: Any = ""
  reasoning_content: str | None = None
  tool_calls: list[ToolCall] | None = None
  observation: Observation | None = None
  metrics: Metrics | None = None
  is_copied_context: bool | None = None
  llm_call_count: int | None = None
  extra: MetadataDict = None

  @pydantic.model_validator(mode="after")
  def _agent_only_fields(self):
    if self.source != Source.AGENT:
      bad = [f for f in _AGENT_ONLY if getattr(self, f) is not None]
      if bad:
        raise ValueError(
            f"fields {bad} are only allowed when source is 'agent', but source"
            f" is '{self.source.value}'")
    return self

  @pydantic.model_validator(mode="after")
  def _observation_matches_calls(self):
    if self.observation is None or not self.tool_calls:
      return self
    ids = {c.tool_call_id for c in self.tool_calls}
    for r in self.observation.results:
      if r.source_call_id is not None and r.source_call_id not in ids:
        raise ValueError(
            f"observation result refers to unknown tool call '{r.source_call_id}'")
    return self


class Agent(_Strict):
  name: str
  version: str = "unknown"
  model_name: str | None = None
  tool_definitions: list[dict[str, Any]] | None = None
  extra: MetadataDict = None


class TrajectoryMetadata(_Strict):
  """Everything about a trajectory except its steps and embedded sub-agents."""

  schema_version: str = SCHEMA_VERSION
  session_id: str | None = None
  trajectory_id: str | None = None
  agent: Agent
  notes: str | None = None
  final_metrics: FinalMetrics | None = None
  continued_trajectory_ref: str | None = None
  extra: MetadataDict = None


def _check_sequential(steps, start):
  steps.sort(key=lambda s: s.step_id)
  for want, s in enumerate(steps, start=start):
    if s.step_id != want:
      raise ValueError(
          f"Expected step_id {want} (sequential from {start}), got {s.step_id}")
  return steps


def _check_subagents(subs):
  if not subs:
    return subs
  seen = set()
  for i, t in enumerate(subs):
    if t.trajectory_id is None:
      raise ValueError(
          f"subagent_trajectories[{i}].trajectory_id is required for embedded"
          " subagents.")
    if t.trajectory_id in seen:
      raise ValueError(
          f"subagent_trajectories[{i}].trajectory_id: duplicate ID"
          f" '{t.trajectory_id}'")
    seen.add(t.trajectory_id)
  return subs


class Trajectory(TrajectoryMetadata):
  """Metadata plus the ordered interaction history (step ids start at 1)."""

  steps: list[Step] = pydantic.Field(default_factory=list)
  subagent_trajectories: list["Trajectory"] | None = None

  _FIRST_STEP_ID = 1

  @pydantic.field_validator("steps")
  @classmethod
  def validate_step_ids(cls, steps):
    return _check_sequential(steps, 1)

  @pydantic.field_validator("subagent_trajectories")
  @classmethod
  def validate_embedded_subagent_trajectory_ids(cls, subs):
    return _check_subagents(subs)

  def add_step(self, source: Source, message: Any = "", *,
               timestamp: datetime.datetime | None = None, **fields) -> Step:
    """Appends a step with the next id and the current UTC time."""
    step = Step(
        step_id=len(self.steps) + 1,
        timestamp=timestamp or datetime.datetime.now(datetime.timezone.utc),
        source=source, message=message, **fields)
    self.steps.append(step)
    return step

  def get_metadata(self) -> TrajectoryMetadata:
    data = self.model_dump(exclude={"steps", "subagent_trajectories"})
    return TrajectoryMetadata.model_validate(data)

  def to_json_dict(self, exclude_none: bool = True) -> dict[str, Any]:
    return self.model_dump(mode="json", exclude_none=exclude_none)

  @classmethod
  def from_json_dict(cls, data: dict[str, Any]):
    return cls.model_validate(data)


# ---------------------------------------------------------------------------
# Token-level extensions for RL.
# ---------------------------------------------------------------------------


class _ArrayStep(Step):
  model_config = pydantic.ConfigDict(arbitrary_types_allowed=True, extra="forbid")


class TunixAgentStep(_ArrayStep):
  """An agent turn with the sampled tokens and the policy that sampled them."""

  mc_return: float | None = None
  assistant_tokens: IntArray = None
  assistant_masks: IntArray = None
  logprobs: FloatArray = None
  policy_version: int | None = None

  @pydantic.model_validator(mode="after")
  def validate_agent_source(self):
    if self.source != Source.AGENT:
      raise ValueError(
          "TunixAgentStep is only applicable when source is 'agent', but source"
          f" is '{self.source.value}'")
    return self

  @pydantic.model_validator(mode="after")
  def _lengths_agree(self):
    n = None if self.assistant_tokens is None else len(self.assistant_tokens)
    for name in ("assistant_masks", "logprobs"):
      v = getattr(self, name)
      if n is not None and v is not None and len(v) != n:
        raise ValueError(
            f"{name} has {len(v)} entries but assistant_tokens has {n}")
    return self


class TunixEnvStep(_ArrayStep):
  """An environment (system or user) turn with its reward and tokens."""

  reward: float | None = None
  done: bool | None = None
  env_tokens: IntArray = None
  env_masks: IntArray = None

  @pydantic.model_validator(mode="after")
  def validate_env_source(self):
    if self.source not in (Source.SYSTEM, Source.USER):
      raise ValueError(
          "TunixEnvStep is only applicable when source is 'system' or 'user',"
          f" but source is '{self.source.value}'")
    return self


class TunixTrajectoryMetadata(TrajectoryMetadata):
  prompt_id: str | None = None
  group_offset_id: str | None = None
  target_policy_versions: list[int] | None = None
  status: str | None = None
  total_reward: float | None = None
  hyperparams: dict[str, Any] | None = None
  env_time: dict[str, float] | None = None
  reward_time: dict[str, float] | None = None


def _parse_tunix_step(v):
  if isinstance(v, Step):
    return v
  if isinstance(v, dict):
    src = v.get("source")
    src = src.value if isinstance(src, Source) else src
    cls = TunixAgentStep if src == Source.AGENT.value else TunixEnvStep
    return cls.model_validate(v)
  return v


TunixStep = Annotated[TunixAgentStep | TunixEnvStep,
                      pydantic.BeforeValidator(_parse_tunix_step)]


class TunixTrajectory(TunixTrajectoryMetadata):
  """RL trajectory; step ids start at 0 and alternate env / agent turns freely."""

  model_config = pydantic.ConfigDict(arbitrary_types_allowed=True, extra="forbid")

  steps: list[TunixStep] = pydantic.Field(default_factory=list)
  subagent_trajectories: list["TunixTrajectory"] | None = None

  @pydantic.field_validator("steps")
  @classmethod
  def validate_step_ids(cls, steps):
    return _check_sequential(steps, 0)

  @pydantic.field_validator("subagent_trajectories")
  @classmethod
  def validate_embedded_subagent_trajectory_ids(cls, subs):
    return _check_subagents(subs)

  def add_step(self, source: Source, message: Any = "", *,
               timestamp: datetime.datetime | None = None,
               reasoning_content=None, tool_calls=None, observation=None,
               metrics=None, model_name=None, reasoning_effort=None,
               is_copied_context=None, llm_call_count=None, reward=None,
               done=None, mc_return=None, assistant_tokens=None,
               assistant_masks=None, env_tokens=None, env_masks=None,
               logprobs=None, policy_version=None,
               extra=None) -> TunixAgentStep | TunixEnvStep:
    """Appends an agent or environment step with the next 0-based id."""
    common = dict(
        step_id=len(self.steps),
        timestamp=timestamp or datetime.datetime.now(datetime.timezone.utc),
        source=source, message=message, observation=observation, extra=extra)
    if source == Source.AGENT:
      step = TunixAgentStep(
          **common, reasoning_content=reasoning_content, tool_calls=tool_calls,
          metrics=metrics, model_name=model_name,
          reasoning_effort=reasoning_effort, is_copied_context=is_copied_context,
          llm_call_count=llm_call_count, mc_return=mc_return,
          assistant_tokens=assistant_tokens, assistant_masks=assistant_masks,
          logprobs=logprobs, policy_version=policy_version)
    else:
      step = TunixEnvStep(**common, reward=reward, done=done,
                          env_tokens=env_tokens, env_masks=env_masks)
    self.steps.append(step)
    return step

  def get_metadata(self) -> TunixTrajectoryMetadata:
    data = self.model_dump(exclude={"steps", "subagent_trajectories"})
    return TunixTrajectoryMetadata.model_validate(data)

  def to_json_dict(self, exclude_none: bool = True) -> dict[str, Any]:
    return self.model_dump(mode="json", exclude_none=exclude_none)

  @classmethod
  def from_json_dict(cls, data: dict[str, Any]):
    return cls.model_validate(data)

  # -- learner-facing views -------------------------------------------------

  def flat_tokens(self):
    """Concatenates per-step tokens and loss masks in step order.

    Environment tokens get mask 0 unless the step carries its own mask; agent
    tokens get mask 1 unless overridden. Returns (tokens, masks, logprobs) as
    int32 / int32 / float32 arrays; log-probs are 0 for environment tokens.
    """
    toks, masks, lps = [], [], []
    for s in self.steps:
      if isinstance(s, TunixAgentStep):
        if s.assistant_tokens is None:
          continue
        n = len(s.assistant_tokens)
        toks.append(s.assistant_tokens)
        masks.append(s.assistant_masks if s.assistant_masks is not None
                     else np.ones(n, np.int32))
        lps.append(s.logprobs if s.logprobs is not None
                   else np.zeros(n, np.float32))
      else:
        if s.env_tokens is None:
          continue
        n = len(s.env_tokens)
        toks.append(s.env_tokens)
        masks.append(s.env_masks if s.env_masks is not None
                     else np.zeros(n, np.int32))
        lps.append(np.zeros(n, np.float32))
    if not toks:
      z = np.zeros(0, np.int32)
      return z, z.copy(), np.zeros(0, np.float32)
    return (np.concatenate(toks).astype(np.int32),
            np.concatenate(masks).astype(np.int32),
            np.concatenate(lps).astype(np.float32))

  def sum_rewards(self) -> float:
    return float(sum(s.reward or 0.0 for s in self.steps
                     if isinstance(s, TunixEnvStep)))


Trajectory.model_rebuild()
TunixTrajectory.model_rebuild()
