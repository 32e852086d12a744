"""GRPO learner (https://arxiv.org/abs/2402.03300), also GSPO-token via `loss_algo`
(tunix/rl/grpo/grpo_learner.py:47-590).

Per global step: sample G completions per prompt, score them with the reward functions,
compute group-relative advantages, optionally the reference log-probabilities (beta != 0) and the
old-policy log-probabilities (from the rollout engine, or recomputed on the trainer side with the
anchor weights), then mu optimisation passes over the batch."""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Iterable, List, Optional, Sequence

import numpy as np
import torch

from ...common.datatypes import Mode, Role
from .. import algo_core  # noqa: F401  (registers losses and advantage estimators)
from .. import algorithm_config as algo_config_lib
from .. import common, function_registry, reward_manager  # noqa: F401
from .. import rl_cluster as rl_engine_lib
from .. import rl_learner
from ..common import TrainExample

TrainingInputT = rl_learner.TrainingInputT
RewardFn = reward_manager.RewardFn


@dataclasses.dataclass(kw_only=True)
class GRPOConfig(algo_config_lib.AlgorithmConfig):
  """`num_generations` G >= 2 samples per prompt; `num_iterations` mu passes per batch; `beta` KL
  coefficient (0 disables the reference model); `epsilon` clip; `loss_algo` "grpo" or
  "gspo-token"; `use_rollout_logps`: take old-policy log-probs from the sampler instead of
  recomputing them; `sampler_is="token"`: truncated importance-sampling correction between
  sampler and trainer with weights capped at `sampler_is_threshold`."""

  algo_variant: str = "grpo"
  advantage_estimator: str = "grpo"
  policy_loss_fn: str = "grpo"
  loss_agg_mode: str = "sequence-mean-token-mean"
  reward_manager: str = "sequence-level"
  loss_algo: str = "grpo"
  num_generations: int = 2
  num_iterations: int = 1
  beta: Optional[float] = 0.04
  kl_loss_mode: str = "kl"
  epsilon: float = 0.2
  use_rollout_logps: bool = True
  sampler_is: Optional[str] = None
  sampler_is_threshold: float = 2.0
  temperature: float = 1.0      # filled from the rollout config by the learner

  def __post_init__(self):
    if self.num_generations <= 1:
      raise ValueError(f"num_generations must be greater than 1. Received: {self.num_generations}")
    if self.loss_algo not in ["grpo", "gspo-token"]:
      raise ValueError(f"loss_algo should be either grpo or gspo-token. Received: {self.loss_algo}")
    if self.sampler_is not in (None, "token"):
      raise ValueError(f"sampler_is should be either None or 'token'. Received: {self.sampler_is}")
    super().__post_init__()


def _masked_stats(rollout_lp: torch.Tensor, trainer_lp: torch.Tensor, mask: torch.Tensor) -> Dict[str, Any]:
  """Agreement between sampler and trainer log-probabilities over completion tokens."""
  m = mask.bool()
  mf = m.float()
  n = mf.sum().clamp(min=1.0)
  diff = (rollout_lp - trainer_lp).abs()
  rp, tp = rollout_lp.exp(), trainer_lp.exp()
  pd = (rp - tp).abs()
  rpm, tpm = (rp * mf).sum() / n, (tp * mf).sum() / n
  rd, td = (rp - rpm) * mf, (tp - tpm) * mf
  cov, rv, tv = (rd * td).sum() / n, (rd * rd).sum() / n, (td * td).sum() / n
  zero = torch.zeros_like(diff)
  return {
      "sampler_trainer/logp_diff_mean": (float((diff * mf).sum() / n), np.mean),
      "sampler_trainer/logp_diff_max": (float(torch.where(m, diff, zero).max()), np.max),
      "sampler_trainer/prob_diff_mean": (float((pd * mf).sum() / n), np.mean),
      "sampler_trainer/prob_diff_max": (float(torch.where(m, pd, zero).max()), np.max),
      "sampler_trainer/probs_pearson_corr": (float(cov / torch.sqrt(torch.clamp(rv * tv, min=1e-12))), np.mean),
  }


class GRPOLearner(rl_learner.RLLearner):

  def __init__(self, rl_engine=None, algo_config: GRPOConfig = None, reward_fns=None,
               metric_fns: Optional[Sequence[Any]] = None, data_shuffle_seed: Optional[int] = None, rl_cluster=None):
    super().__init__(rl_engine=rl_engine, algo_config=algo_config, reward_fns=reward_fns, metric_fns=metric_fns,
                     data_shuffle_seed=data_shuffle_seed, rl_cluster=rl_cluster)
    self.algo_config.temperature = self.rl_engine.get_rollout_config(Mode.TRAIN).temperature
    policy_loss_fn = function_registry.get_policy_loss_fn(self.algo_config.policy_loss_fn)
    tc = self.rl_engine.cluster_config.training_config

    def loss_fn(model, train_example, algo_config):
      dev = next(model.parameters()).device
      return policy_loss_fn(model, train_example.to_tensors(dev), algo_config=self.algo_config,
                            pad_id=self.rl_engine.rollout.pad_id(), eos_id=self.rl_engine.rollout.eos_id(),
                            compute_logps_chunk_size=tc.compute_logps_chunk_size)

    if self.algo_config.use_rollout_logps and self.algo_config.sampler_is != "token":
      # the old-policy log-probs come from the sampler: nothing reads the start-of-step snapshot of the weights
      self.rl_engine.snapshot_anchor_on_sync = False
    tr = self.rl_engine.actor_trainer
    tr.with_loss_fn(loss_fn, has_aux=True)
    tr.with_gen_model_input_fn(lambda x: {"train_example": x, "algo_config": self.algo_config})
    tr.with_rl_metrics_to_log({"kl": np.mean, "pg_clipfrac": np.mean, "sampler_is/weight_mean": np.mean,
                               "sampler_is/weight_min": np.min})
    tr.with_tqdm_metrics_to_display([lambda: "kl" if self.algo_config.beta not in (None, 0.0) else None])

  def _generate_and_compute_advantage(self, training_input: TrainingInputT, mode: Mode = Mode.TRAIN) -> TrainExample:
    eng = self.rl_engine
    cfg = self.algo_config
    rc = eng.get_rollout_config(mode)
    training_input["prompts"] = list(training_input["prompts"])
    pad, eos = eng.rollout.pad_id(), eng.rollout.eos_id()
    G = cfg.num_generations
    out = eng.generate(prompts=training_input["prompts"], mode=mode,
                       micro_batch_size=self._rollout_micro_batch_size * G, trace_tags={"step": eng.global_steps})
    L = rc.max_tokens_to_generate
    comp = np.stack([common.pad_to_length(np.asarray(t), L, pad)[:L] for t in out.tokens]).astype(np.int64)
    prompt_ids = torch.from_numpy(np.asarray(out.left_padded_prompt_tokens)).long()
    prompt_mask = prompt_ids != pad
    completion_ids = torch.from_numpy(comp)
    completion_mask = completion_ids != pad
    logps_mb = self._compute_logps_micro_batch_size * G if self._compute_logps_micro_batch_size else len(
        training_input["prompts"])
    ref_lp = None
    if cfg.beta not in (None, 0.0):
      with eng.perf.span("refer_inference", _devs(eng, Role.REFERENCE)) as sp:
        ref_lp = eng.get_ref_per_token_logps(prompt_ids, completion_ids, pad, eos, micro_batch_size=logps_mb).cpu()
        sp.device_end([ref_lp])
    rollout_lp = trainer_lp = old_lp = sis = None
    if cfg.use_rollout_logps and out.logprobs is not None:
      rollout_lp = torch.from_numpy(np.stack([
          common.pad_to_length(np.asarray(l, dtype=np.float32), L, 0)[:L] for l in out.logprobs]))
      old_lp = rollout_lp
    if (not cfg.use_rollout_logps) or cfg.sampler_is == "token":
      with eng.perf.span("old_actor_inference", _devs(eng, Role.ACTOR)) as sp:
        trainer_lp = eng.get_actor_per_token_logps(prompt_ids, completion_ids, pad, eos,
                                                   micro_batch_size=logps_mb).cpu()
        sp.device_end([trainer_lp])
    if not cfg.use_rollout_logps:
      old_lp = trainer_lp
    elif cfg.sampler_is == "token" and trainer_lp is not None:
      old_lp = trainer_lp
    if cfg.num_iterations > 1 and old_lp is None:
      raise RuntimeError("old_per_token_logps is not available for off-policy RL. Enable `return_logprobs` in "
                         "RolloutConfig.")
    with eng.perf.span("advantage_computation"):
      extra = {k: v for k, v in training_input.items() if k != "prompts"}
      rewards = self._compute_rewards(prompts=training_input["prompts"], completions=out.text, mode=mode, **extra)
      advantages = function_registry.get_advantage_estimator(cfg.advantage_estimator)(
          rewards=rewards, num_generations=G)
    eng.buffer_metrics({"rewards/score/mean": (np.mean(rewards), np.mean), "rewards/score/max": (np.max(rewards), np.max),
                        "rewards/score/min": (np.min(rewards), np.min)}, mode=mode)
    lens = completion_mask.sum(-1).numpy()
    eng.buffer_metrics({"completions/mean_length": (np.mean(lens), np.mean),
                        "completions/max_length": (np.max(lens), np.max),
                        "completions/min_length": (np.min(lens), np.min)}, mode=mode)
    if rollout_lp is not None and trainer_lp is not None:
      eng.buffer_metrics(_masked_stats(rollout_lp, trainer_lp, completion_mask), mode=mode)
      if cfg.sampler_is == "token":
        mf = completion_mask.float()
        lr = torch.clamp(trainer_lp - rollout_lp, -20.0, 20.0)
        sis = (torch.clamp(lr.exp(), max=cfg.sampler_is_threshold) * mf).detach()
        n = mf.sum().clamp(min=1.0)
        eng.buffer_metrics({
            "sampler_is/weight_mean": (float((sis * mf).sum() / n), np.mean),
            "sampler_is/weight_max": (float(torch.where(mf > 0, sis, torch.zeros_like(sis)).max()), np.max),
            "sampler_is/frac_clipped_at_threshold": (
                float((((lr.exp() > cfg.sampler_is_threshold) & (mf > 0)).float()).sum() / n), np.mean)}, mode=mode)
    for fn in self.metric_fns:
      eng.buffer_metrics(fn(prompts=training_input["prompts"], completions=out.text, advantages=advantages,
                            rewards=rewards, **extra), mode=mode)
    return TrainExample(prompt_ids=prompt_ids, prompt_mask=prompt_mask, completion_ids=completion_ids,
                        completion_mask=completion_mask, ref_per_token_logps=ref_lp,
                        advantages=torch.as_tensor(np.asarray(advantages), dtype=torch.float32),
                        old_per_token_logps=old_lp, sampler_is_weights=sis)

  def _compute_trajectory_ids(self, example: TrainingInputT, steps: int) -> List[str]:
    """`{row}_{group index}` for every sample of the (already xG repeated) batch."""
    G = self.algo_config.num_generations
    bs = len(example["prompts"]) // G
    rows = np.repeat(np.arange(steps * bs, steps * bs + bs), G)
    groups = np.tile(np.arange(G), bs)
    return [f"{r}_{g}" for r, g in zip(rows, groups)]

  def _num_iterations(self) -> int:
    return self.algo_config.num_iterations

  def _num_generations(self) -> int:
    return self.algo_config.num_generations


def _devs(eng, role):
  m = eng.r2m.get(role)
  return m.ranks() if m is not None else None


GrpoConfig = GRPOConfig
GrpoLearner = GRPOLearner
