"""Compute primitives an RL program is written against
(tunix/experimental/orchestrator/rl_engine_interface.py:25-130)."""
from __future__ import annotations

from typing import Any, List, Mapping, Optional, Protocol, Sequence, runtime_checkable

from ..common import datatypes
from ..worker import remote_execution


@runtime_checkable
class AbstractRLEngine(Protocol):
  async def dispatch_rollout_requests(self, requests: Sequence[datatypes.RolloutRequest]) -> List[str]: ...

  async def dispatch_rollouts(self, prompts: Sequence[Any], *, group_size: int = 1, policy_version: int = 0,
                              generation_args: Optional[datatypes.GenerationArgs] = None,
                              route_metadata: Optional[Mapping[str, Any]] = None, **kwargs: Any) -> List[str]:
    """Every prompt needs a unique `prompt_id`; each is expanded into `group_size` requests with
    ids `req_{prompt_id}_{g}_v{version}` and `pair_index = g`."""

  async def poll_rollouts(self, timeout_s: float = remote_execution.LONG_POLL_TIMEOUT_S
                          ) -> List[datatypes.TrajectoryItem]: ...

  async def generate(self, prompts: Sequence[Any], generation_args: Optional[datatypes.GenerationArgs] = None,
                     route_metadata: Optional[Mapping[str, Any]] = None, **kwargs: Any
                     ) -> List[datatypes.TrajectoryItem]: ...

  async def score(self, role: datatypes.Role, items: Sequence[Any], **kwargs: Any) -> List[float]: ...

  async def per_token_logps(self, role: datatypes.Role, items: Any, **kwargs: Any) -> Any: ...

  async def train_step(self, payload: Any, role: datatypes.Role = datatypes.Role.ACTOR,
                       accumulate_gradients: bool = False, apply_optimizer: bool = True, skip_jit: bool = False,
                       **kwargs: Any) -> Any: ...

  async def sync_weights(self, role: datatypes.Role = datatypes.Role.ACTOR,
                         target_roles: Optional[Sequence[datatypes.Role]] = None, **kwargs: Any) -> int: ...
