"""GRPO over multi-turn agent trajectories (tunix/rl/agentic/agentic_grpo_learner.py:62-885).

A group is the `num_generations` episodes of one prompt. The prompt is left-padded to
`max_prompt_length`; everything after it (assistant turns and environment turns interleaved)
is the "completion", right-padded to `max_response_length`, and the completion mask is 1 on
assistant tokens only, so environment text conditions the policy but is never trained on.
Old log-probs come from the rollout engine (or a trainer recompute), reference log-probs when
`beta != 0` (or `force_compute_kl`), rewards from the reward manager plus the environment's
trajectory reward, advantages from the registered estimator.
"""
from __future__ import annotations

import dataclasses
import logging
from typing import Any, Dict, List, Optional, Sequence, Tuple, Type, TypeVar

import numpy as np
import torch

from ...common.datatypes import Mode, Role
from .. import common, function_registry, utils as rl_utils
from . import agentic_rl_learner, utils as agentic_utils
from .agents import base_agent, model_agent
from .environments import base_environment, task_environment

TrainExample = agentic_rl_learner.TrainExample


@dataclasses.dataclass(kw_only=True)
class GRPOConfig(agentic_rl_learner.AgenticRLConfig):
  algo_variant: str = "agentic_grpo"
  advantage_estimator: str = "grpo"
  policy_loss_fn: str = "grpo"
  loss_agg_mode: str = "sequence-mean-token-mean"
  loss_algo: str = "grpo"                 # "grpo" | "gspo-token"
  num_generations: int = 2
  num_iterations: int = 1
  beta: float = 0.04
  kl_loss_mode: str = "kl"
  force_compute_kl: bool = False
  epsilon: float = 0.2
  epsilon_high: Optional[float] = None     # DAPO uses 0.28
  system_prompt: str = ""
  max_concurrency: int = 16
  off_policy_steps: int = 0
  degenerate_group_masking: bool = False
  use_rollout_logps: bool = True
  sampler_is: Optional[str] = None         # None | "token"
  sampler_is_threshold: float = 2.0
  temperature: float = 1.0

  def __post_init__(self):
    if self.num_generations <= 1:
      raise ValueError(f"num_generations must be greater than 1. Received: {self.num_generations}")
    if self.epsilon_high is None:
      self.epsilon_high = self.epsilon
    if self.loss_algo not in ("grpo", "gspo-token"):
      raise ValueError(f"loss_algo should be either grpo or gspo-token. Received: {self.loss_algo}")


TGrpoConfig = TypeVar("TGrpoConfig", bound=GRPOConfig)


def sampler_trainer_agreement(rollout_lp: Optional[torch.Tensor], trainer_lp: Optional[torch.Tensor],
                              completion_mask: torch.Tensor, sampler_is: Optional[str], threshold: float
                              ) -> Tuple[Dict[str, Any], Optional[torch.Tensor]]:
  """Agreement metrics between the rollout engine's and the trainer's log-probs of the sampled
  tokens, and the truncated importance weights min(exp(trainer - rollout), threshold)."""
  if rollout_lp is None or trainer_lp is None:
    return {}, None
  rollout_lp, trainer_lp = rollout_lp.float(), trainer_lp.float().to(rollout_lp.device)
  mask = completion_mask.to(rollout_lp.device).bool()
  mf = mask.float()
  n = mf.sum().clamp(min=1.0)
  diff = (rollout_lp - trainer_lp).abs()
  rp, tp = rollout_lp.exp(), trainer_lp.exp()
  pdiff = (rp - tp).abs()
  rp_d = (rp - (rp * mf).sum() / n) * mf
  tp_d = (tp - (tp * mf).sum() / n) * mf
  cov, rv, tv = (rp_d * tp_d).sum() / n, (rp_d * rp_d).sum() / n, (tp_d * tp_d).sum() / n
  zero = torch.zeros_like(diff)
  metrics = {
      "sampler_trainer/logp_diff_mean": (float((diff * mf).sum() / n), np.mean),
      "sampler_trainer/logp_diff_max": (float(torch.where(mask, diff, zero).max()), np.max),
      "sampler_trainer/prob_diff_mean": (float((pdiff * mf).sum() / n), np.mean),
      "sampler_trainer/prob_diff_max": (float(torch.where(mask, pdiff, zero).max()), np.max),
      "sampler_trainer/probs_pearson_corr": (float(cov / torch.sqrt(torch.clamp(rv * tv, min=1e-12))), np.mean),
  }
  weights = None
  if sampler_is == "token":
    lr = torch.clamp(trainer_lp - rollout_lp, -20.0, 20.0)
    ratio = lr.exp()
    weights = (torch.clamp(ratio, max=threshold) * mf).detach()
    metrics.update({
        "sampler_is/weight_mean": (float((weights * mf).sum() / n), np.mean),
        "sampler_is/weight_max": (float(torch.where(mask, weights, zero).max()), np.max),
        "sampler_is/frac_clipped_at_threshold": (float(((ratio > threshold) & mask).float().sum() / n), np.mean)})
  return metrics, weights


class GRPOLearner(agentic_rl_learner.AgenticRLLearner[TGrpoConfig]):
  def __init__(self, rl_engine=None, algo_config: GRPOConfig = None, reward_fns=None, chat_parser: Any = None,
               metric_fns: Optional[Sequence[Any]] = None,
               agent_class: Type[base_agent.ConversationAgentBase] = model_agent.ModelAgent,
               agent_kwargs: Optional[Dict[str, Any]] = None,
               env_class: Type[base_environment.BaseTaskEnv] = task_environment.TaskEnvironment,
               env_kwargs: Optional[Dict[str, Any]] = None, rl_cluster=None):
    super().__init__(rl_engine=rl_engine, algo_config=algo_config, reward_fns=reward_fns, chat_parser=chat_parser,
                     metric_fns=metric_fns, agent_class=agent_class, agent_kwargs=agent_kwargs, env_class=env_class,
                     env_kwargs=env_kwargs, rl_cluster=rl_cluster)
    eng = self.rl_engine
    self._trajectory_logger = None
    opts = eng.cluster_config.training_config.metrics_logging_options
    log_dir = getattr(opts, "log_dir", None) if opts else None
    if log_dir:
      from ...utils import trajectory_logger
      self._trajectory_logger = trajectory_logger.AsyncTrajectoryLogger(log_dir)
    else:
      logging.warning("Metrics log dir is None, skipping trajectory logging.")
    self.algo_config.temperature = eng.get_rollout_config(Mode.TRAIN).temperature
    policy_loss_fn = function_registry.get_policy_loss_fn(self.algo_config.policy_loss_fn)
    tc = eng.cluster_config.training_config

    def loss_fn(model, train_example, algo_config):
      dev = next(model.parameters()).device
      return policy_loss_fn(model, train_example.to_tensors(dev), algo_config=self.algo_config,
                            pad_id=eng.rollout.pad_id(), eos_id=eng.rollout.eos_id(),
                            compute_logps_chunk_size=tc.compute_logps_chunk_size)
    tr = eng.actor_trainer
    tr.with_loss_fn(loss_fn, has_aux=True)
    tr.with_gen_model_input_fn(lambda x: {"train_example": x, "algo_config": self.algo_config})
    mm, gw = common.mean_of_means, common.global_weighted_mean
    tr.with_rl_metrics_to_log({
        "kl": mm, "entropy": mm, "reduced_pg_loss": mm, "unreduced_pg_loss": gw, "pg_clipfrac": mm, "ppo_kl": mm,
        "kl_loss": mm, "is_ratio/mean": mm, "is_ratio/max": np.max, "is_ratio/min": np.min, "log_ratio/abs_mean": mm,
        "pg_loss/unclipped_mean": mm, "pg_loss/clipped_mean": mm, "advantage/abs_mean": mm, "advantage/max": np.max,
        "advantage/min": np.min, "advantage/nonzero_frac": mm, "sampler_is/weight_mean": mm,
        "sampler_is/weight_min": np.min})
    tr.with_tqdm_metrics_to_display(
        [lambda: "kl" if self.algo_config.force_compute_kl or self.algo_config.beta != 0.0 else None])

  def _have_actor_mesh(self) -> bool:
    mesh = self.rl_engine.cluster_config.role_to_mesh.get(Role.ACTOR)
    return mesh is not None and getattr(mesh, "size", 1) >= 1

  def _needs_kl(self) -> bool:
    return bool(self.algo_config.force_compute_kl or self.algo_config.beta not in (None, 0.0))

  def _sampler_trainer_agreement(self, rollout_lp, trainer_lp, completion_mask):
    return sampler_trainer_agreement(rollout_lp, trainer_lp, completion_mask, self.algo_config.sampler_is,
                                     self.algo_config.sampler_is_threshold)

  def _compute_packed_logps(self, example: TrainExample) -> TrainExample:
    """Packed rows: log-probs are computed after packing ("pack first"), on the packed layout."""
    eng, cfg = self.rl_engine, self.algo_config
    pad, eos = eng.rollout.pad_id(), eng.rollout.eos_id()
    micro = eng.cluster_config.training_config.compute_logps_micro_batch_size
    kw = dict(prompt_tokens=torch.as_tensor(example.prompt_ids), completion_tokens=torch.as_tensor(example.completion_ids),
              pad_id=pad, eos_id=eos, micro_batch_size=micro, segment_ids=example.segment_ids,
              segment_positions=example.segment_positions)
    updates: Dict[str, Any] = {}
    if example.old_per_token_logps is None and not cfg.use_rollout_logps:
      updates["old_per_token_logps"] = eng.get_actor_per_token_logps(**kw)
    if example.ref_per_token_logps is None and self._needs_kl():
      updates["ref_per_token_logps"] = eng.get_ref_per_token_logps(**kw)
    if cfg.use_rollout_logps and example.old_per_token_logps is not None and (
        self._have_actor_mesh() or cfg.sampler_is == "token"):
      rollout_lp = torch.as_tensor(example.old_per_token_logps)
      trainer_lp = eng.get_actor_per_token_logps(**kw)
      metrics, weights = self._sampler_trainer_agreement(rollout_lp, trainer_lp.cpu(),
                                                         torch.as_tensor(example.completion_mask))
      if metrics:
        eng.buffer_metrics_async(metrics, mode=Mode.TRAIN, step=eng.global_steps)
      if weights is not None:
        updates["sampler_is_weights"] = weights
        updates["old_per_token_logps"] = trainer_lp
    return dataclasses.replace(example, **updates) if updates else example

  # ---- a group of trajectories -> TrainExample -----------------------------------------------
  def _process_results(self, trajectories: List[Any], mode: Mode = Mode.TRAIN,
                       expected_step: Optional[int] = None) -> List[TrainExample]:
    eng, cfg = self.rl_engine, self.algo_config
    pad, eos = eng.rollout.pad_id(), eng.rollout.eos_id()
    rc = eng.get_rollout_config(mode)
    L = cfg.max_response_length
    texts, versions, traj_rewards, raw_lens = [], [], [], []
    p_ids, c_ids, c_masks, old_lps = [], [], [], []
    clipped = 0
    for item in trajectories:
      t = item.traj
      if self._trajectory_logger is not None:
        self._trajectory_logger.log_item_async(t)
      conv = t.get("conversation_text") or []
      texts.append(next((m["content"] for m in conv if m["role"] == "assistant"), ""))
      if t.get("policy_version") is None:
        raise ValueError("policy_version is missing from trajectory task.")
      versions.append(t["policy_version"])
      traj_rewards.append(t.get("trajectory_reward"))
      toks, mask, olp = t.get("conversation_tokens"), t.get("conversation_masks"), t.get("old_logprobs")
      raw_lens.append(min(len(toks), L))
      if len(toks) >= L and len(mask) and mask[-1] != eos:
        clipped += 1
      pp, cc, _ = agentic_utils.pad_prompt_and_completion(t.get("prompt_tokens"), toks, rc.max_prompt_length, L, pad)
      p_ids.append(pp)
      c_ids.append(cc[:L])
      c_masks.append(agentic_utils.right_pad(mask, L, 0)[:L])
      if cfg.use_rollout_logps:
        old_lps.append(agentic_utils.right_pad(olp, L, 0.0, dtype=np.float32)[:L] if olp is not None
                       else np.zeros(L, np.float32))
    prompt_ids = torch.from_numpy(np.stack(p_ids)).long()
    prompt_mask = prompt_ids != pad
    completion_ids = torch.from_numpy(np.stack(c_ids)).long()
    completion_mask = torch.from_numpy(np.stack(c_masks)).bool()
    tc = eng.cluster_config.training_config
    is_packed = tc.max_seq_token_per_tpu is not None
    mb = tc.compute_logps_micro_batch_size * cfg.num_generations if tc.compute_logps_micro_batch_size else len(trajectories)
    logp_kw = dict(prompt_tokens=prompt_ids, completion_tokens=completion_ids, pad_id=pad, eos_id=eos,
                   micro_batch_size=mb)
    rollout_lp = trainer_lp = old_lp = None
    if cfg.use_rollout_logps and old_lps:
      rollout_lp = old_lp = torch.from_numpy(np.stack(old_lps))
      if (self._have_actor_mesh() or cfg.sampler_is == "token") and not is_packed:
        trainer_lp = eng.get_actor_per_token_logps(**logp_kw).cpu()
      if cfg.sampler_is == "token" and trainer_lp is not None:
        old_lp = trainer_lp
    elif not cfg.use_rollout_logps and not is_packed:
      trainer_lp = old_lp = eng.get_actor_per_token_logps(**logp_kw).cpu()
    if cfg.num_iterations > 1 and old_lp is None:
      raise RuntimeError("old_per_token_logps is not available for off-policy RL. Enable `return_logprobs` in "
                         "RolloutConfig.")
    ref_lp = eng.get_ref_per_token_logps(**logp_kw).cpu() if self._needs_kl() and not is_packed else None

    originals = rl_utils.merge_micro_batches([item.traj["original_input"] for item in trajectories])
    reward_kw = {k: v for k, v in originals.items() if k != "prompts"}
    reward_kw["trajectory_rewards"] = traj_rewards
    rewards = self._compute_rewards(prompts=originals["prompts"], completions=texts, mode=mode,
                                    expected_step=expected_step, **reward_kw)
    advantages = function_registry.get_advantage_estimator(cfg.advantage_estimator)(
        rewards=rewards, num_generations=cfg.num_generations)
    adv = np.asarray(advantages, dtype=np.float32)
    if cfg.degenerate_group_masking:
      grp = adv.reshape(-1, cfg.num_generations)
      dead = np.repeat(np.all(grp == 0, axis=1), cfg.num_generations)
      completion_mask = completion_mask & torch.from_numpy(~dead)[:, None]

    lens = completion_mask.sum(-1).numpy()
    plen = len(trajectories[0].traj.get("prompt_tokens"))
    raw = np.asarray(raw_lens)
    metrics = {
        "generation/prompts/mean_length": (plen, np.mean), "generation/prompts/max_length": (plen, np.max),
        "generation/prompts/min_length": (plen, np.min),
        "generation/completions/mean_length": (lens.mean(), np.mean),
        "generation/completions/max_length": (lens.max(), np.max),
        "generation/completions/min_length": (lens.min(), np.min),
        "generation/completions/mean_raw_length": (raw.mean(), np.mean),
        "generation/completions/max_raw_length": (raw.max(), np.max),
        "generation/completions/min_raw_length": (raw.min(), np.min),
        "generation/completions/clip_ratio": (clipped / len(trajectories), np.mean),
        "rewards/advantage/mean": (adv.mean(), np.mean), "rewards/advantage/max": (adv.max(), np.max),
        "rewards/advantage/min": (adv.min(), np.min), "rewards/advantage/std": (adv.std(), np.mean)}
    agree, sis = self._sampler_trainer_agreement(rollout_lp, trainer_lp, completion_mask)
    metrics.update(agree)
    for key in ("env_time", "reward_time"):
      dicts = [item.traj.get(key, {}) or {} for item in trajectories]
      for sub in {k for d in dicts for k in d}:
        flat: List[float] = []
        for d in dicts:
          v = d.get(sub, 0.0)
          flat.extend(v if isinstance(v, (list, tuple, np.ndarray)) else ([] if v is None else [v]))
        flat = flat or [0.0]
        metrics.update({f"trajectory/{key}/{sub}/mean": (np.mean(flat), np.mean),
                        f"trajectory/{key}/{sub}/max": (np.max(flat), np.max)})
    statuses = [item.traj.get("status") for item in trajectories]
    for name in set(statuses):
      metrics[f"trajectory/status/{name}"] = (statuses.count(name) / len(statuses), np.mean)
    eng.buffer_metrics_async(metrics, mode=mode, step=expected_step or 0)
    for fn in self.metric_fns:
      eng.buffer_metrics_async(fn(prompts=originals["prompts"], completions=texts, advantages=advantages,
                                  rewards=rewards, **{k: v for k, v in reward_kw.items() if k != "trajectory_rewards"}),
                               mode=mode, step=expected_step or 0)
    return [TrainExample(prompt_ids=prompt_ids, prompt_mask=prompt_mask, completion_ids=completion_ids,
                         completion_mask=completion_mask, advantages=torch.from_numpy(adv), ref_per_token_logps=ref_lp,
                         old_per_token_logps=old_lp, sampler_is_weights=sis,
                         policy_version=np.asarray(versions, dtype=np.int32))]
