"""What an RL program may ask of a cluster (tunix/experimental/orchestrator/rl_engine_interface.py:25-130).

The contract is an abstract base class, not a structural protocol: the part every engine would otherwise
repeat - turning a list of prompts into `group_size` rollout requests each, with stable ids - lives here
(`GroupExpansion`), and engines only implement transport: where a request goes, how results come back, how a
role trains, scores and receives weights.
"""
from __future__ import annotations

import abc
import dataclasses
from typing import Any, Dict, Iterator, List, Mapping, Optional, Sequence

from ..common import datatypes
from ..worker import remote_execution


def request_id(prompt_id: str, sample: int, version: int) -> str:
  """Id of sample `sample` of a prompt at a policy version. Results are matched back to groups by it."""
  return f"req_{prompt_id}_{sample}_v{version}"


@dataclasses.dataclass
class GroupExpansion:
  """Expands prompt items into rollout requests: one group per prompt, `group_size` samples per group.

  A prompt item is a mapping or an object with at least `prompt_id` (unique among prompts in flight) and
  `prompt`; optional `group_id`, `metadata`, `generation_kwargs`, `max_turns`. Ready-made `RolloutRequest`s pass
  through. All samples of a group share `prefix_hash` (the routing key), so they reach the same worker and can
  share the prompt's KV pages; `env_config`, when present, is stamped with the group, the sample index and the
  policy version.
  """
  group_size: int = 1
  policy_version: int = 0
  generation: Dict[str, Any] = dataclasses.field(default_factory=dict)
  metadata: Dict[str, Any] = dataclasses.field(default_factory=dict)
  default_max_turns: int = 10

  @staticmethod
  def _field(item: Any, name: str, default: Any = None) -> Any:
    return item.get(name, default) if isinstance(item, Mapping) else getattr(item, name, default)

  def _sample_metadata(self, item_md: Mapping[str, Any], group: str, sample: int) -> Dict[str, Any]:
    md = {**self.metadata, **item_md, "group_id": group, "pair_index": sample}
    md.setdefault("prefix_hash", group)
    env = md.get("env_config")
    if isinstance(env, Mapping):
      md["env_config"] = {"group_id": group, **env, "pair_index": sample, "policy_version": self.policy_version}
    return md

  def requests(self, prompts: Sequence[Any]) -> Iterator[datatypes.RolloutRequest]:
    for position, item in enumerate(prompts):
      if isinstance(item, datatypes.RolloutRequest):
        yield item
        continue
      pid = self._field(item, "prompt_id")
      if not pid:
        raise ValueError(f"Prompt at index {position} lacks 'prompt_id'. Every prompt item dispatched to an engine "
                         "must provide a unique, collision-free 'prompt_id' (as an attribute or dict key).")
      pid = str(pid)
      item_md = dict(self._field(item, "metadata") or {})
      group = str(self._field(item, "group_id") or item_md.get("group_id") or pid)
      text = self._field(item, "prompt", item)
      own_generation = dict(self._field(item, "generation_kwargs") or {})
      for sample in range(self.group_size):
        yield datatypes.RolloutRequest(
            request_id=request_id(pid, sample, self.policy_version), prompt=text, prompt_id=pid,
            group_offset_id=str(sample), target_policy_version=self.policy_version,
            generation_kwargs={**self.generation, **own_generation},
            max_turns=self._field(item, "max_turns", self.default_max_turns),
            metadata=self._sample_metadata(item_md, group, sample))


class AbstractRLEngine(abc.ABC):
  """Primitives of the control plane. Calls are coroutines; an engine may serve them in process or over RPC."""

  # ---- rollouts: fire-and-collect
  @abc.abstractmethod
  async def dispatch_rollout_requests(self, requests: Sequence[datatypes.RolloutRequest]) -> List[str]:
    """Hands fully formed requests to rollout workers; returns their ids without waiting for results."""

  async def dispatch_rollouts(self, prompts: Sequence[Any], *, group_size: int = 1, policy_version: int = 0,
                              generation_args: Optional[datatypes.GenerationArgs] = None,
                              route_metadata: Optional[Mapping[str, Any]] = None, **kwargs: Any) -> List[str]:
    """Expands every prompt into `group_size` requests (`GroupExpansion`) and dispatches them."""
    plan = GroupExpansion(
        group_size=group_size, policy_version=kwargs.get("policy_version", policy_version),
        generation=generation_args.as_kwargs() if generation_args else {},
        metadata={**(route_metadata or {}), **(kwargs.get("metadata") or {})})
    return await self.dispatch_rollout_requests(list(plan.requests(prompts)))

  @abc.abstractmethod
  async def poll_rollouts(self, timeout_s: float = remote_execution.LONG_POLL_TIMEOUT_S
                          ) -> List[datatypes.TrajectoryItem]:
    """Finished rollouts since the last poll (waits up to `timeout_s` for the first)."""

  # ---- rollouts: call-and-wait
  @abc.abstractmethod
  async def generate(self, prompts: Sequence[Any], generation_args: Optional[datatypes.GenerationArgs] = None,
                     route_metadata: Optional[Mapping[str, Any]] = None, **kwargs: Any
                     ) -> List[datatypes.TrajectoryItem]:
    """Synchronous generation for evaluation and simple programs."""

  # ---- scoring and training by role
  @abc.abstractmethod
  async def score(self, role: datatypes.Role, items: Sequence[Any], **kwargs: Any) -> List[float]:
    """Scalar scores (reward or value model) of `items`."""

  @abc.abstractmethod
  async def per_token_logps(self, role: datatypes.Role, items: Any, **kwargs: Any) -> Any:
    """Per-token log-probabilities of the completions under `role`'s model."""

  @abc.abstractmethod
  async def train_step(self, payload: Any, role: datatypes.Role = datatypes.Role.ACTOR,
                       accumulate_gradients: bool = False, apply_optimizer: bool = True, skip_jit: bool = False,
                       **kwargs: Any) -> Any:
    """One micro-step (or a full step) on `role`'s trainer."""

  @abc.abstractmethod
  async def sync_weights(self, role: datatypes.Role = datatypes.Role.ACTOR,
                         target_roles: Optional[Sequence[datatypes.Role]] = None, **kwargs: Any) -> int:
    """Publishes `role`'s weights to the target roles; returns the new policy version."""
