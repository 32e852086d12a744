"""Worker-backed implementation of the engine interface
(tunix/experimental/orchestrator/distributed_rl_engine.py:36-423): rollout requests are routed by
prefix (samples of one prompt land on one worker, which can share their prompt KV pages),
trainer / inference calls go to the role's handle, weight sync to the coordinator."""
from __future__ import annotations

import asyncio
import collections
from typing import Any, Dict, List, Mapping, Optional, Sequence

import numpy as np

from ..common import datatypes
from ..worker import remote_execution
from . import rl_engine_interface


def _response_to_trajectory_item(resp: Any) -> datatypes.TrajectoryItem:
  if isinstance(resp, datatypes.TrajectoryItem):
    return resp
  if isinstance(resp, dict):
    resp = datatypes.RolloutResponse(**resp)
  toks, mask, lps = resp.completion()
  md = dict(resp.metadata or {})
  md["old_logps"] = lps
  md["status"] = resp.status
  if resp.error is not None:
    md["error"] = resp.error.message
  traj = datatypes.Trajectory(reward=resp.env_reward)
  return datatypes.TrajectoryItem(
      pair_index=int(md.get("pair_index", 0)), group_id=md.get("group_id", resp.prompt_id), start_step=0, traj=traj,
      metadata=md, prompt_tokens=np.asarray(resp.prompt_tokens), completion_tokens=toks, action_mask=mask,
      policy_version=resp.policy_version)


def _role_name(role: Any) -> Any:
  return getattr(role, "value", role)


class DistributedRLEngine(rl_engine_interface.AbstractRLEngine):
  def __init__(self, rollout_workers: Sequence[remote_execution.ActorHandle],
               trainer_workers: Mapping[Any, remote_execution.ActorHandle],
               inference_workers: Optional[Mapping[Any, remote_execution.ActorHandle]] = None,
               weight_sync_coordinator: Any = None):
    self._rollout_workers = list(rollout_workers)
    self._rollout_pool = remote_execution.RoutingActorPool(self._rollout_workers)
    # roles are looked up by their plain name, so `Role.ACTOR` and "actor" name the same worker on either side
    self._trainer_workers = {_role_name(k): v for k, v in dict(trainer_workers).items()}
    self._inference_workers = {_role_name(k): v for k, v in dict(inference_workers or {}).items()}
    self._policy_version = 0
    self._weight_sync_coordinator = weight_sync_coordinator

  @property
  def policy_version(self) -> int:
    return self._policy_version

  def _route(self, key) -> remote_execution.ActorHandle:
    return self._rollout_pool._get_next_actor(kwargs={"route_key": key} if key is not None else {})

  async def dispatch_rollout_requests(self, requests) -> List[str]:
    for r in requests:
      worker = self._route((r.metadata or {}).get("prefix_hash", r.prompt_id))
      await worker.dispatch_task(r.request_id, "generate", requests=[r])
    return [r.request_id for r in requests]

  async def poll_rollouts(self, timeout_s: float = remote_execution.LONG_POLL_TIMEOUT_S):
    if not self._rollout_workers:
      return []
    batches = await asyncio.gather(*[w.poll_responses(timeout_s=timeout_s) for w in self._rollout_workers],
                                   return_exceptions=True)
    done: List[datatypes.TrajectoryItem] = []
    for b in batches:
      if isinstance(b, BaseException) or not b:
        continue
      for resp in b:
        res = resp.unwrap() if hasattr(resp, "unwrap") else resp
        for it in (res if isinstance(res, list) else [res]):
          if it is not None:
            done.append(_response_to_trajectory_item(it))
    return done

  async def generate(self, prompts, generation_args=None, route_metadata=None, **kwargs):
    if not self._rollout_workers:
      raise ValueError("DistributedRLEngine has no registered rollout workers.")
    if kwargs:
      raise TypeError(f"Unexpected generate kwargs: {sorted(kwargs)}. Use generation_args=GenerationArgs(...) for "
                      "sampling parameters.")
    gen = generation_args.as_kwargs() if generation_args is not None else {}
    rmd = dict(route_metadata or {})
    by_worker: Dict[int, Any] = collections.OrderedDict()
    for p in prompts:
      if isinstance(p, datatypes.RolloutRequest):
        key, field = (p.metadata or {}).get("prefix_hash", p.prompt_id), "requests"
      else:
        key, field = rmd.get("prefix_hash", rmd.get("prompt_id")), "prompts"
      w = self._route(key)
      by_worker.setdefault(id(w), (w, {"requests": [], "prompts": []}))[1][field].append(p)
    calls = []
    for w, groups in by_worker.values():
      for field, items in groups.items():
        if items:
          calls.append(w.asubmit("generate", **{field: items}, **gen))
    out: List[datatypes.TrajectoryItem] = []
    for res in await asyncio.gather(*calls):
      out += [_response_to_trajectory_item(r) for r in (res if isinstance(res, list) else [res])]
    return out

  def _inference(self, role):
    w = self._inference_workers.get(_role_name(role))
    if w is None:
      raise ValueError(f"no inference worker registered for role {role}")
    return w

  async def score(self, role, items, **kwargs) -> List[float]:
    res = await self._inference(role).asubmit("score", items=items, **kwargs)
    return list(getattr(res, "scores", res))

  async def per_token_logps(self, role, items, **kwargs):
    res = await self._inference(role).asubmit("per_token_logps", items=items, **kwargs)
    return getattr(res, "per_token_logps", res)

  async def train_step(self, payload, role=datatypes.Role.ACTOR, accumulate_gradients: bool = False,
                       apply_optimizer: bool = True, skip_jit: bool = False, **kwargs):
    w = self._trainer_workers.get(_role_name(role))
    if w is None:
      raise ValueError(f"no trainer worker registered for role {role}")
    return await w.asubmit("train_step", payload=payload, accumulate_gradients=accumulate_gradients,
                           apply_optimizer=apply_optimizer, **kwargs)

  async def sync_weights(self, role=datatypes.Role.ACTOR, target_roles=None, **kwargs) -> int:
    """One coordinated round to version current+1; returns the new policy version."""
    new_version = self._policy_version + 1
    if self._weight_sync_coordinator is not None:
      await self._weight_sync_coordinator.sync(new_version)
    self._policy_version = new_version
    return new_version
