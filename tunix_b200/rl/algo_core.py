"""Advantage estimators and loss functions of the RL algorithms, registered by name:
`advantage_estimator/{gae,grpo,rloo,drgrpo}`, `policy_loss_fn/{ppo,grpo}`, `value_loss_fn/ppo`.
Math follows tunix/rl/algo_core.py:33-707."""
from __future__ import annotations

from typing import Any, Optional, Tuple

import numpy as np
import torch

from ..sft import utils as sft_utils
from . import common
from . import function_registry as registry

WeightedMetric = sft_utils.WeightedMetric
LossOutput = sft_utils.LossOutput


def masked_mean(x: torch.Tensor, mask: torch.Tensor, axis: Optional[int] = None) -> torch.Tensor:
  m = mask.to(x.dtype)
  if axis is None:
    return (x * m).sum() / (m.sum() + 1e-8)
  return (x * m).sum(axis) / (m.sum(axis) + 1e-8)


def masked_var(x: torch.Tensor, mask: torch.Tensor, mean: Optional[torch.Tensor] = None) -> torch.Tensor:
  """Masked variance with Bessel's correction."""
  m = mask.to(x.dtype)
  if mean is None:
    mean = masked_mean(x, m)
  var = masked_mean((x - mean) ** 2, m)
  n = m.sum()
  return var * (n / (n - 1))


def masked_whiten(x: torch.Tensor, completion_mask: torch.Tensor) -> torch.Tensor:
  mean = masked_mean(x, completion_mask)
  var = masked_var(x, completion_mask, mean)
  return (x - mean) * torch.rsqrt(var + 1e-8)


@registry.register_advantage_estimator("gae")
def compute_gae_advantages(rewards: torch.Tensor, values: torch.Tensor, completion_mask: torch.Tensor, gamma: float,
                           gae_lambda: float) -> Tuple[torch.Tensor, torch.Tensor]:
  """Generalised advantage estimation with a reverse scan over time that skips masked steps
  (`delta_t = r_t + gamma V_{t+1} - V_t`, `A_t = delta_t + gamma lambda A_{t+1}`), then masked
  whitening. Returns (advantages, returns = unwhitened advantages + values)."""
  rewards = torch.as_tensor(rewards, dtype=torch.float32)
  values = torch.as_tensor(values, dtype=torch.float32, device=rewards.device)
  mask = torch.as_tensor(completion_mask, dtype=torch.float32, device=rewards.device)
  B, T = values.shape
  gae = torch.zeros(B, device=rewards.device)
  next_values = torch.zeros(B, device=rewards.device)
  adv = torch.zeros_like(values)
  for t in range(T - 1, -1, -1):
    delta = rewards[:, t] + gamma * next_values - values[:, t]
    gae_t = delta + gamma * gae_lambda * gae
    next_values = values[:, t] * mask[:, t] + (1 - mask[:, t]) * next_values
    gae = gae_t * mask[:, t] + (1 - mask[:, t]) * gae
    adv[:, t] = gae
  returns = adv + values
  return masked_whiten(adv, mask), returns


@registry.register_advantage_estimator("grpo")
def compute_advantages(rewards: np.ndarray, num_generations: int) -> np.ndarray:
  """Group-relative advantages `(r - mean_g) / (std_g(ddof=1) + 1e-6)`."""
  r = np.asarray(rewards, dtype=np.float32)
  g = r.reshape(-1, num_generations)
  mean = g.mean(axis=-1).repeat(num_generations)
  with np.errstate(invalid="ignore", divide="ignore"):
    std = g.std(axis=-1, ddof=1).repeat(num_generations) if num_generations > 1 else np.full_like(r, np.nan)
  return (r - mean) / (std + 1e-6)


@registry.register_advantage_estimator("rloo")
def compute_rloo_advantages(rewards, num_generations: int):
  """Leave-one-out baseline: each completion against the mean reward of its group's others."""
  r = np.asarray(rewards, dtype=np.float32)
  if num_generations < 2:
    return np.zeros_like(r)
  g = r.reshape(-1, num_generations)
  loo = (g.sum(axis=-1, keepdims=True) - g) / (num_generations - 1)
  return (g - loo).reshape(-1)


@registry.register_advantage_estimator("drgrpo")
def compute_drgrpo_advantages(rewards, num_generations: int):
  """Dr. GRPO: `r - mean_g`, no division by the standard deviation."""
  r = np.asarray(rewards, dtype=np.float32)
  return r - r.reshape(-1, num_generations).mean(axis=1).repeat(num_generations)


def _get(obj, name, default=None):
  return getattr(obj, name, default)


@registry.register_policy_loss_fn("ppo")
def ppo_policy_loss_fn(model, train_example, algo_config, pad_id, eos_id, **kwargs) -> LossOutput:
  """Clipped PPO policy loss with optional dual clip (`epsilon_c`), entropy bonus and in-loss KL."""
  eps_low, eps_high = algo_config.epsilon_low, algo_config.epsilon_high
  entropy_coef = _get(algo_config, "entropy_coef")
  mask = train_example.completion_mask.float()
  want_ent = entropy_coef is not None and entropy_coef != 0.0
  out = common.compute_per_token_logps(
      model, train_example.prompt_ids, train_example.completion_ids, pad_id, eos_id, stop_gradient=False,
      return_entropy=want_ent, segment_ids=_get(train_example, "segment_ids"),
      segment_positions=_get(train_example, "segment_positions"))
  logps, ent = out if want_ent else (out, None)
  adv = train_example.advantages
  ratio = torch.exp(logps - train_example.old_per_token_logps)
  l1 = -ratio * adv
  l2 = -torch.clamp(ratio, 1 - eps_low, 1 + eps_high) * adv
  ptl = torch.maximum(l1, l2)
  eps_c = _get(algo_config, "epsilon_c")
  l3 = -eps_c * adv if eps_c is not None else ptl
  clipfrac_lower = (((ptl > l3) & (adv < 0.0)).float() * mask).sum()
  pg = torch.where(adv < 0.0, torch.minimum(l3, ptl), ptl)
  denom = mask.sum()
  clipfrac = ((l2 > l1).float() * mask).sum()
  loss = (pg * mask).sum()
  aux = {"pg_clipfrac": WeightedMetric(clipfrac, denom, min_denom=1.0),
         "pg_clipfrac_lower": WeightedMetric(clipfrac_lower, denom, min_denom=1.0)}
  if want_ent:
    e = (ent * mask).sum()
    loss = loss - entropy_coef * e
    aux["loss/entropy"] = WeightedMetric(e, denom, min_denom=1.0)
  kl_coef = _get(algo_config, "kl_coef", 0.0) or 0.0
  if kl_coef > 0.0 and train_example.ref_per_token_logps is not None:
    kl = common.compute_kl_divergence(logps, train_example.ref_per_token_logps, "kl",
                                      clamp_value=_get(algo_config, "kl_clamp_value"))
    k = (kl * mask).sum()
    loss = loss + kl_coef * k
    aux["kl"] = WeightedMetric(k, denom, min_denom=1.0)
  return LossOutput(primary_loss=WeightedMetric(loss, denom, min_denom=1.0), aux_metrics=aux)


@registry.register_value_loss_fn("ppo")
def ppo_value_loss_fn(model, train_example, clip_range_value: Optional[float], pad_id: int, eos_id: int) -> LossOutput:
  """`0.5 * max((v - R)^2, (clip(v, v_old +- c) - R)^2)` averaged over completion tokens."""
  mask = train_example.completion_mask.float()
  values, returns = train_example.old_values, train_example.returns
  seg = _get(train_example, "segment_ids")
  keep = train_example.completion_ids.shape[1] - (1 if seg is not None else 0)
  vpreds = common.compute_score(model, train_example.prompt_ids, train_example.completion_ids, pad_id, eos_id,
                                stop_gradient=False, segment_ids=seg,
                                segment_positions=_get(train_example, "segment_positions"))
  vpreds = vpreds[:, -keep - 1:-1].float()
  if seg is not None:
    vpreds = torch.nn.functional.pad(vpreds, (1, 0))
  vclip = torch.clamp(vpreds, values - clip_range_value, values + clip_range_value) if clip_range_value else vpreds
  v1, v2 = (vpreds - returns) ** 2, (vclip - returns) ** 2
  denom = mask.sum()
  primary = WeightedMetric(0.5 * (torch.maximum(v1, v2) * mask).sum(), denom, min_denom=1.0)
  aux = {"vf_loss": primary,
         "vpred_mean": WeightedMetric((vpreds * mask).sum(), denom, min_denom=1.0),
         "vf_clipfrac": WeightedMetric(((v2 > v1).float() * mask).sum(), denom, min_denom=1.0),
         "return_mean": WeightedMetric((returns * mask).sum(), denom, min_denom=1.0)}
  return LossOutput(primary_loss=primary, aux_metrics=aux)


@registry.register_policy_loss_fn("grpo")
def grpo_loss_fn(model, train_example, algo_config, pad_id, eos_id, **kwargs) -> LossOutput:
  """GRPO / GSPO-token policy loss.

  log-ratio = logp - old_logp (old = detached logp when none is given), clipped to +-20;
  GSPO-token replaces the per-token ratio by the sequence (segment) mean ratio with a per-token
  gradient path, clipped at 10; `pg = max(-A r, -A clip(r, 1 - eps, 1 + eps_high))`; dual clip
  with `epsilon_c` on negative advantages; optional sampler importance weights; aggregation by
  `loss_agg_mode`; `+ beta * aggregate(kl)` when beta != 0."""
  beta, epsilon, loss_algo = algo_config.beta, algo_config.epsilon, algo_config.loss_algo
  eps_high = _get(algo_config, "epsilon_high", epsilon)
  eps_high = epsilon if eps_high is None else eps_high
  eps_c = _get(algo_config, "epsilon_c")
  mode = algo_config.loss_agg_mode
  mask = train_example.completion_mask.float()
  seg, nseg = _get(train_example, "segment_ids"), _get(train_example, "num_segments")
  logps, ent = common.compute_per_token_logps(
      model, train_example.prompt_ids, train_example.completion_ids, pad_id, eos_id, stop_gradient=False,
      return_entropy=True, segment_ids=seg, segment_positions=_get(train_example, "segment_positions"),
      temperature=_get(algo_config, "temperature", 1.0))
  logps = logps.float()
  adv = torch.as_tensor(train_example.advantages, device=logps.device).float()
  old = logps.detach() if train_example.old_per_token_logps is None else train_example.old_per_token_logps.float()
  log_ratio = logps - old
  token_denom = mask.sum()
  ppo_kl = (-log_ratio * mask).sum()
  log_ratio = torch.clamp(log_ratio, -20.0, 20.0)
  if loss_algo == "gspo-token":
    if seg is None:
      seq_mean = ((log_ratio * mask).sum(-1) / mask.sum(-1).clamp(min=1)).unsqueeze(-1)
    else:
      per_seg = common.segmented_sum(log_ratio * mask, seg, nseg) / common.segmented_count(seg, nseg, mask).clamp(min=1.0)
      seq_mean = per_seg.gather(1, seg.long())
    log_ratio = torch.clamp(logps - logps.detach() + seq_mean.detach(), max=10.0)
  ratio = torch.exp(log_ratio)
  a = adv if adv.dim() == 2 else adv.unsqueeze(1)
  l1 = -a * ratio
  l2 = -a * torch.clamp(ratio, 1 - epsilon, 1 + eps_high)
  ptl = torch.maximum(l1, l2).float()
  clip_frac = ((l2 > l1).float() * mask).sum()
  l3 = -eps_c * a if eps_c is not None else ptl
  agg = lambda x: common.aggregate_loss(x, mask, mode, segment_ids=seg, num_segments=nseg)
  clipfrac_lower = agg(((ptl > l3) & (a < 0.0)).float())
  ptl = torch.where(a < 0.0, torch.minimum(l3, ptl), ptl)
  sis = _get(train_example, "sampler_is_weights")
  if sis is not None:
    ptl = ptl * sis.float()
  pg = agg(ptl)
  total = pg
  with torch.no_grad():
    reduced = common.reduced_loss_agg(ptl, mask, mode, segment_ids=seg, num_segments=nseg)
    ab = a.expand_as(mask)
    inf = torch.tensor(float("inf"), device=mask.device)
    aux = {
        "kl": WeightedMetric(torch.tensor(0.0), torch.tensor(1.0)),
        "kl_loss": WeightedMetric(torch.tensor(0.0), torch.tensor(1.0)),
        "reduced_pg_loss": reduced,
        "unreduced_pg_loss": pg.detach(),
        "pg_clipfrac": WeightedMetric(clip_frac, token_denom, min_denom=1.0),
        "ppo_kl": WeightedMetric(ppo_kl.detach(), token_denom, min_denom=1.0),
        "pg_clipfrac_lower": clipfrac_lower,
        "is_ratio/mean": masked_mean(ratio, mask),
        "is_ratio/max": torch.where(mask > 0, ratio, torch.zeros_like(ratio)).max(),
        "is_ratio/min": torch.where(mask > 0, ratio, inf).min(),
        "log_ratio/abs_mean": masked_mean(log_ratio.abs(), mask),
        "pg_loss/unclipped_mean": masked_mean(l1, mask),
        "pg_loss/clipped_mean": masked_mean(l2, mask),
        "advantage/abs_mean": masked_mean(ab.abs(), mask),
        "advantage/max": torch.where(mask > 0, ab, -inf).max(),
        "advantage/min": torch.where(mask > 0, ab, inf).min(),
        "advantage/nonzero_frac": masked_mean((ab.abs() > 1e-8).float(), mask),
    }
    if sis is not None:
      aux["sampler_is/weight_mean"] = masked_mean(sis.float(), mask)
      aux["sampler_is/weight_min"] = torch.where(mask > 0, sis.float(), inf).min()
    else:
      aux["sampler_is/weight_mean"] = torch.tensor(1.0)
      aux["sampler_is/weight_min"] = torch.tensor(1.0)
  kl_loss = None
  if train_example.ref_per_token_logps is not None:
    kl = common.compute_kl_divergence(logps, train_example.ref_per_token_logps, algo_config.kl_loss_mode,
                                      clamp_value=_get(algo_config, "kl_clamp_value"))
    aux["kl"] = WeightedMetric((kl * mask).sum().detach().float(), token_denom, min_denom=1.0)
    kl_loss = agg(kl)
    aux["kl_loss"] = kl_loss.detach()
  if beta is not None and beta != 0.0:
    if kl_loss is None:
      raise ValueError("beta != 0 requires ref_per_token_logps")
    total = WeightedMetric(pg.unreduced_sum + beta * kl_loss.unreduced_sum, pg.denominator, eps=pg.eps,
                           min_denom=pg.min_denom)
  aux["entropy"] = agg(ent.detach())
  return LossOutput(primary_loss=total, aux_metrics=aux)
