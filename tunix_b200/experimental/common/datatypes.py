"""Wire-level data types of the control plane (tunix/experimental/common/datatypes.py:43-590).
Everything here is primitives and numpy arrays, so it pickles across process boundaries."""
from __future__ import annotations

import dataclasses
import enum
import time
from typing import Any, Dict, List, Optional

import numpy as np

from ...common.datatypes import Role  # noqa: F401  (roles of the control plane are the cluster roles)
from ...rl.agentic.agents import agent_types

Trajectory = agent_types.Trajectory


@dataclasses.dataclass(kw_only=True)
class TrajectoryItem(agent_types.TrajectoryItem):
  prompt_tokens: Optional[np.ndarray] = None
  completion_tokens: Optional[np.ndarray] = None
  action_mask: Optional[np.ndarray] = None
  policy_version: int = 0


@dataclasses.dataclass(kw_only=True)
class ErrorInfo:
  """A failure reported in-band on a response."""
  error_type: str
  message: str
  retryable: bool = False
  traceback: str = ""

  @classmethod
  def from_exception(cls, e: BaseException, retryable: bool = False) -> "ErrorInfo":
    import traceback as tb
    return cls(error_type=type(e).__name__, message=str(e), retryable=retryable,
               traceback="".join(tb.format_exception(type(e), e, e.__traceback__)))


@dataclasses.dataclass(kw_only=True)
class Request:
  request_id: str = ""
  metadata: Dict[str, Any] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(kw_only=True)
class Response:
  request_id: str = ""
  error: Optional[ErrorInfo] = None
  metadata: Dict[str, Any] = dataclasses.field(default_factory=dict)

  @property
  def ok(self) -> bool:
    return self.error is None


class WorkerState(str, enum.Enum):
  PENDING = "PENDING"
  INITIALIZING = "INITIALIZING"
  COMPILING = "COMPILING"
  READY = "READY"
  SYNCING = "SYNCING"
  DRAINING = "DRAINING"
  STOPPED = "STOPPED"
  ERROR = "ERROR"

  def can_transition_to(self, new_state: "WorkerState") -> bool:
    return new_state in _ALLOWED_TRANSITIONS.get(self, frozenset())


_S = WorkerState
_ALLOWED_TRANSITIONS = {
    _S.PENDING: frozenset({_S.INITIALIZING, _S.STOPPED, _S.ERROR}),
    _S.INITIALIZING: frozenset({_S.READY, _S.STOPPED, _S.ERROR}),
    _S.COMPILING: frozenset({_S.READY, _S.STOPPED, _S.ERROR}),
    _S.READY: frozenset({_S.COMPILING, _S.SYNCING, _S.DRAINING, _S.STOPPED, _S.ERROR}),
    _S.SYNCING: frozenset({_S.READY, _S.STOPPED, _S.ERROR}),
    _S.DRAINING: frozenset({_S.STOPPED, _S.ERROR}),
    _S.STOPPED: frozenset(),
    _S.ERROR: frozenset({_S.STOPPED}),
}


@dataclasses.dataclass(kw_only=True)
class HealthReport:
  state: WorkerState
  inflight: int = 0
  queue_depth: int = 0
  policy_version: int = 0
  last_error: Optional[str] = None
  heartbeat_unix_s: float = dataclasses.field(default_factory=time.time)


@dataclasses.dataclass(kw_only=True)
class WorkerInfo:
  worker_id: str
  roles: frozenset = frozenset()
  resources: Dict[str, Any] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(frozen=True, kw_only=True)
class GenerationArgs:
  max_generation_steps: Optional[int] = None
  temperature: Optional[float] = None
  top_p: Optional[float] = None
  top_k: Optional[int] = None
  seed: Optional[int] = None
  return_logprobs: Optional[bool] = None

  def as_kwargs(self) -> Dict[str, Any]:
    return {f.name: getattr(self, f.name) for f in dataclasses.fields(self) if getattr(self, f.name) is not None}


@dataclasses.dataclass(kw_only=True)
class RolloutRequest(Request):
  prompt: Any = ""
  prompt_id: str = "default_prompt"
  group_offset_id: str = ""
  generation_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)
  max_turns: int = 10
  target_policy_version: int = 0

  @property
  def traj_id(self) -> str:
    return f"traj_{self.prompt_id}_{self.group_offset_id}" if self.group_offset_id else f"traj_{self.prompt_id}"


@dataclasses.dataclass(kw_only=True)
class TokenSegment:
  """One turn of the token stream: `source` is "assistant" (sampled, trainable) or "env"."""
  source: str
  tokens: np.ndarray
  loss_mask: np.ndarray
  logps: Optional[np.ndarray] = None

  def __post_init__(self):
    if self.loss_mask.shape != self.tokens.shape:
      raise ValueError(f"loss_mask shape {self.loss_mask.shape} != tokens shape {self.tokens.shape}")
    if self.logps is not None and self.logps.shape != self.tokens.shape:
      raise ValueError(f"logps shape {self.logps.shape} != tokens shape {self.tokens.shape}")


@dataclasses.dataclass(kw_only=True)
class RolloutResponse(Response):
  prompt_id: str = ""
  status: str
  prompt_tokens: np.ndarray = dataclasses.field(default_factory=lambda: np.zeros(0, np.int32))
  segments: List[TokenSegment] = dataclasses.field(default_factory=list)
  env_reward: float = 0.0
  policy_version: int = 0

  @classmethod
  def from_trajectory(cls, traj: Any, request_id: str = "", prompt_id: str = "", policy_version: int = 0
                      ) -> "RolloutResponse":
    """Wire form of an agent `Trajectory`: token spans only, no message text or live objects."""
    segs: List[TokenSegment] = []
    for step in getattr(traj, "steps", []):
      a = getattr(step, "assistant_tokens", None)
      if a is not None and len(a):
        lp = getattr(step, "logprobs", None)
        segs.append(TokenSegment(source="assistant", tokens=np.asarray(a), loss_mask=np.asarray(step.assistant_masks),
                                 logps=np.asarray(lp) if lp is not None else None))
      e = getattr(step, "env_tokens", None)
      if e is not None and len(e):
        segs.append(TokenSegment(source="env", tokens=np.asarray(e), loss_mask=np.asarray(step.env_masks)))
    status = getattr(traj, "status", None)
    pt = getattr(traj, "prompt_tokens", None)
    return cls(request_id=request_id, prompt_id=prompt_id, status=getattr(status, "name", str(status or "UNKNOWN")),
               prompt_tokens=np.asarray(pt if pt is not None else [], dtype=np.int32), segments=segs,
               env_reward=float(getattr(traj, "reward", 0.0) or 0.0), policy_version=policy_version)

  def completion(self):
    """-> (tokens, loss_mask, logps) concatenated over segments (logps 0 where not sampled)."""
    if not self.segments:
      z = np.zeros(0, np.int32)
      return z, z, np.zeros(0, np.float32)
    toks = np.concatenate([s.tokens for s in self.segments])
    mask = np.concatenate([s.loss_mask for s in self.segments])
    lps = np.concatenate([s.logps if s.logps is not None else np.zeros(len(s.tokens), np.float32)
                          for s in self.segments]).astype(np.float32)
    return toks, mask, lps


@dataclasses.dataclass(kw_only=True)
class WeightSyncRequest(Request):
  controller_id: str = ""
  policy_version: int = 0
  source_metadata: Any = None
  extra_config: Dict[str, Any] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass
class WeightSyncMetadata:
  """Who talks to whom in a decentralised weight transfer (bytes never pass the orchestrator)."""
  worker_ips: List[str] = dataclasses.field(default_factory=list)
  data_ports: List[str] = dataclasses.field(default_factory=list)
  ctrl_ports: List[str] = dataclasses.field(default_factory=list)
  mesh: Any = None
  layout: List[int] = dataclasses.field(default_factory=list)
  new_policy_version: int = 0
  transfer_mode: str = "p2p"
  source_endpoints: List[str] = dataclasses.field(default_factory=list)
  sharding_topology: Dict[str, Any] = dataclasses.field(default_factory=dict)

  def __post_init__(self):
    if self.transfer_mode in ("broadcast", "fs"):
      raise NotImplementedError(f"transfer_mode='{self.transfer_mode}' is not implemented yet. Currently only 'p2p' "
                                "is supported.")
    if self.transfer_mode != "p2p":
      raise ValueError(f"Unknown transfer_mode: {self.transfer_mode!r}")


@dataclasses.dataclass(kw_only=True)
class TrainerPayload:
  token_ids: Any
  token_mask: Any
  segment_ids: Any = None
  segment_positions: Any = None


@dataclasses.dataclass(kw_only=True)
class RLTrainerPayload(TrainerPayload):
  advantages: Any
  loss_mask: Any
  action_mask: Any = None
  prompt_ids: Any = None
  prompt_mask: Any = None
  completion_ids: Any = None
  completion_mask: Any = None
  ref_per_token_logps: Any = None
  old_per_token_logps: Any = None
  sampler_is_weights: Any = None
  returns: Any = None
  old_values: Any = None
  metadata: Dict[str, Any] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(kw_only=True)
class LogprobsRequest(Request):
  prompt_tokens: np.ndarray            # [B, P] left-padded
  completion_tokens: np.ndarray        # [B, C] right-padded
  temperature: float
  model_role: str = "reference"


@dataclasses.dataclass(kw_only=True)
class LogprobsResponse(Response):
  per_token_logps: np.ndarray
  model_version: int = 0


@dataclasses.dataclass(kw_only=True)
class ScoreRequest(Request):
  prompt_tokens: np.ndarray
  completion_tokens: np.ndarray
  model_role: str = "reward"


@dataclasses.dataclass(kw_only=True)
class ScoreResponse(Response):
  scores: np.ndarray
  model_version: int = 0
