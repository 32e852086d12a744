"""Algorithm-specific pieces of the RL program (tunix/experimental/orchestrator/algorithm_adapter.py:32-260):
advantages from a group's rewards, unbatched `RLTrainerPayload`s per trajectory, and the loss
function the trainer worker runs."""
from __future__ import annotations

import abc
from typing import Any, Callable, List, Optional, Sequence

import numpy as np

from ...rl import algo_core, function_registry
from ..common import datatypes


def _payload(item, adv: float, ref_lp=None, returns=None, old_values=None) -> datatypes.RLTrainerPayload:
  p = np.asarray(item.prompt_tokens if item.prompt_tokens is not None else [], dtype=np.int32).reshape(-1)
  c = np.asarray(item.completion_tokens if item.completion_tokens is not None else [], dtype=np.int32).reshape(-1)
  act = np.asarray(item.action_mask if item.action_mask is not None else np.ones(len(c)), dtype=np.float32).reshape(-1)
  toks = np.concatenate([p, c])
  loss_mask = np.concatenate([np.zeros(len(p), np.float32), act])
  meta = dict(getattr(item, "metadata", None) or {})
  old = meta.get("old_logps")
  return datatypes.RLTrainerPayload(
      token_ids=toks, token_mask=np.ones(len(toks), np.float32), loss_mask=loss_mask,
      advantages=np.full(len(toks), adv, np.float32), action_mask=loss_mask, prompt_ids=p,
      prompt_mask=np.ones(len(p), np.float32), completion_ids=c, completion_mask=act,
      ref_per_token_logps=np.asarray(ref_lp, np.float32) if ref_lp is not None else None,
      old_per_token_logps=np.asarray(old, np.float32) if old is not None else None,
      returns=returns, old_values=old_values,
      metadata={"policy_version": getattr(item, "policy_version", 0), "group_id": getattr(item, "group_id", None)})


class AlgorithmAdapter(abc.ABC):
  requires_reference_kl = False

  def __init__(self, group_size: int = 8, mini_batch_size: int = 4, max_turns: int = 1, max_packed_len: int = 8192):
    self.group_size, self.mini_batch_size = group_size, mini_batch_size
    self.max_turns, self.max_packed_len = max_turns, max_packed_len

  @abc.abstractmethod
  def compute_advantages(self, rewards, **kwargs) -> np.ndarray: ...

  @abc.abstractmethod
  def create_trainer_payloads(self, group: Sequence[datatypes.TrajectoryItem], rewards: Sequence[float],
                              ref_logps: Any = None, **kwargs) -> List[datatypes.RLTrainerPayload]: ...

  @abc.abstractmethod
  def loss_fn(self) -> Callable[..., Any]: ...


class GRPOAdapter(AlgorithmAdapter):
  def __init__(self, group_size: int = 8, mini_batch_size: int = 4, max_turns: int = 1, max_packed_len: int = 8192,
               clip_epsilon: float = 0.2, beta_kl: float = 0.04):
    super().__init__(group_size, mini_batch_size, max_turns, max_packed_len)
    self.clip_epsilon, self.beta_kl = clip_epsilon, beta_kl
    self.requires_reference_kl = beta_kl != 0.0

  def compute_advantages(self, rewards, num_generations: Optional[int] = None, **kwargs) -> np.ndarray:
    """(r - mean(group)) / (std(group) + 1e-6), population std."""
    g = num_generations or self.group_size
    r = np.asarray(rewards, dtype=np.float32).reshape(-1, g)
    return ((r - r.mean(-1, keepdims=True)) / (r.std(-1, keepdims=True) + 1e-6)).reshape(-1)

  def create_trainer_payloads(self, group, rewards, ref_logps=None, **kwargs):
    advs = self.compute_advantages(rewards, num_generations=len(group) if len(group) != self.group_size else None)
    return [_payload(item, float(advs[i]), ref_logps[i] if ref_logps is not None and i < len(ref_logps) else None)
            for i, item in enumerate(group)]

  def loss_fn(self) -> Callable[..., Any]:
    return function_registry.get_policy_loss_fn("grpo")


class PPOAdapter(AlgorithmAdapter):
  def __init__(self, group_size: int = 1, mini_batch_size: int = 4, max_turns: int = 1, max_packed_len: int = 8192,
               gamma: float = 1.0, gae_lambda: float = 0.95, clip_epsilon: float = 0.2, beta_kl: float = 0.0):
    super().__init__(group_size, mini_batch_size, max_turns, max_packed_len)
    self.gamma, self.gae_lambda, self.clip_epsilon, self.beta_kl = gamma, gae_lambda, clip_epsilon, beta_kl
    self.requires_reference_kl = beta_kl != 0.0

  def compute_advantages(self, rewards, values=None, mask=None, **kwargs):
    """GAE over per-token rewards [B, T] given values [B, T]; -> (advantages, returns)."""
    import torch
    r = torch.as_tensor(np.asarray(rewards, np.float32))
    v = torch.as_tensor(np.asarray(values, np.float32)) if values is not None else torch.zeros_like(r)
    m = torch.as_tensor(np.asarray(mask, np.float32)) if mask is not None else torch.ones_like(r)
    adv, ret = algo_core.compute_gae_advantages(r, v, m, self.gamma, self.gae_lambda)
    return adv.numpy(), ret.numpy()

  def create_trainer_payloads(self, group, rewards, ref_logps=None, values=None, **kwargs):
    out = []
    for i, item in enumerate(group):
      c = np.asarray(item.completion_tokens if item.completion_tokens is not None else [], np.int32).reshape(-1)
      act = np.asarray(item.action_mask if item.action_mask is not None else np.ones(len(c)), np.float32).reshape(-1)
      tok_r = np.zeros(len(c), np.float32)
      if len(c):
        last = int(np.nonzero(act)[0][-1]) if act.any() else len(c) - 1
        tok_r[last] = float(rewards[i])            # sequence reward on the last trained token
      v = np.asarray(values[i], np.float32) if values is not None else np.zeros(len(c), np.float32)
      adv, ret = self.compute_advantages(tok_r[None], values=v[None], mask=act[None])
      p = _payload(item, 0.0, ref_logps[i] if ref_logps is not None else None, returns=ret[0], old_values=v)
      p.advantages = np.concatenate([np.zeros(len(p.prompt_ids), np.float32), adv[0]])
      out.append(p)
    return out

  def loss_fn(self) -> Callable[..., Any]:
    return function_registry.get_policy_loss_fn("ppo")
