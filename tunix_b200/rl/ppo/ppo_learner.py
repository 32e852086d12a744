"""PPO learner (https://arxiv.org/abs/1707.06347) with an actor, a critic and either a reward
model or reward functions (tunix/rl/ppo/ppo_learner.py:49-543).

Per batch: generate one completion per prompt; old log-probs from the rollout model; values
from the critic; the sequence score is placed on the last valid completion token and
`beta * KL(old || ref)` is subtracted per token; GAE (gamma, lambda) with masked whitening gives
advantages and returns; the actor minimises the clipped surrogate (dual clip, entropy bonus
optional), the critic the clipped value loss."""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ...common.datatypes import Mode
from .. import algo_core  # noqa: F401
from .. import algorithm_config as algo_config_lib
from .. import common, function_registry, rl_learner
from ..algo_core import masked_mean

TrainingInputT = rl_learner.TrainingInputT


@dataclasses.dataclass(frozen=True)
class TrainExample(common.TrainExample):
  returns: Any = None
  old_values: Any = None


@dataclasses.dataclass(kw_only=True)
class PPOConfig(algo_config_lib.AlgorithmConfig):
  algo_variant: str = "ppo"
  advantage_estimator: str = "gae"
  policy_loss_fn: str = "ppo"
  value_loss_fn: str = "ppo"
  reward_manager: str = "sequence-level"
  num_iterations: int = 1
  gamma: float = 1.0
  gae_lambda: float = 0.95
  beta: float = 0.04
  epsilon: float = 0.2
  epsilon_low: Optional[float] = None
  epsilon_high: Optional[float] = None
  epsilon_c: Optional[float] = None
  entropy_coef: Optional[float] = None
  clip_range_value: float = 0.2
  kl_method: str = "low_var_kl"
  kl_coef: float = 0.0

  def __post_init__(self):
    self.epsilon_low = self.epsilon_low if self.epsilon_low else self.epsilon
    self.epsilon_high = self.epsilon_high if self.epsilon_high else self.epsilon
    if self.epsilon_c is not None and self.epsilon_c <= 1.0:
      raise ValueError(f"`epsilon_c` must be greater than 1. Received: {self.epsilon_c}.")
    if self.kl_method not in ["kl", "mse_kl", "low_var_kl"]:
      raise ValueError(f"Invalid KL method: {self.kl_method}. Must be one of ['low_var_kl', 'kl', 'mse_kl'].")
    super().__post_init__()


class PPOLearner(rl_learner.RLLearner):

  def __init__(self, rl_engine=None, algo_config: PPOConfig = None, reward_fns=None,
               metric_fns: Optional[Sequence[Any]] = None, data_shuffle_seed: Optional[int] = None, rl_cluster=None):
    eng = rl_engine if rl_engine is not None else rl_cluster
    models = eng.inference_worker._models
    if bool(reward_fns) == bool(models.get("reward")):
      raise ValueError("PPO requires one of `reward_fns` or `rl_engine.reward` to be set. Received: "
                       f"reward_fn={reward_fns}, rl_engine.reward={models.get('reward')}")
    if not models.get("critic") and not hasattr(eng, "_critic_trainer"):
      raise ValueError("PPO requires a critic model. Please pass the correct `critic` to `RLEngine`.")
    self._use_reward_model = bool(models.get("reward"))
    super().__init__(rl_engine=eng, algo_config=algo_config,
                     reward_fns=reward_fns if reward_fns else [lambda prompts, completions, **kw: [0.0] * len(prompts)],
                     metric_fns=metric_fns, data_shuffle_seed=data_shuffle_seed)
    policy_loss_fn = function_registry.get_policy_loss_fn(self.algo_config.policy_loss_fn)
    value_loss_fn = function_registry.get_value_loss_fn(self.algo_config.value_loss_fn)
    tc = eng.cluster_config.training_config

    def actor_loss(model, train_example, algo_config):
      dev = next(model.parameters()).device
      return policy_loss_fn(model, train_example.to_tensors(dev), algo_config, pad_id=eng.rollout.pad_id(),
                            eos_id=eng.rollout.eos_id(), compute_logps_chunk_size=tc.compute_logps_chunk_size)

    def critic_loss(model, train_example, clip_range_value, pad_id, eos_id):
      dev = next(model.parameters()).device
      return value_loss_fn(model, train_example.to_tensors(dev), clip_range_value, pad_id, eos_id)

    eng.actor_trainer.with_loss_fn(actor_loss, has_aux=True)
    eng.actor_trainer.with_gen_model_input_fn(lambda x: {"train_example": x, "algo_config": self.algo_config})
    eng.critic_trainer.with_loss_fn(critic_loss, has_aux=True)
    eng.critic_trainer.with_gen_model_input_fn(lambda x: {
        "train_example": x, "clip_range_value": self.algo_config.clip_range_value, "pad_id": eng.rollout.pad_id(),
        "eos_id": eng.rollout.eos_id()})
    log_m = {"pg_clipfrac": common.mean_of_means}
    if self.algo_config.epsilon_c is not None:
      log_m["pg_clipfrac_lower"] = common.mean_of_means
    if self.algo_config.entropy_coef:
      log_m["loss/entropy"] = common.mean_of_means
    eng.actor_trainer.with_rl_metrics_to_log(log_m)
    eng.critic_trainer.with_rl_metrics_to_log({"vpred_mean": common.mean_of_means,
                                               "vf_clipfrac": common.mean_of_means})

  def _generate_and_compute_advantage(self, training_input: TrainingInputT, mode: Mode = Mode.TRAIN) -> TrainExample:
    eng, cfg = self.rl_engine, self.algo_config
    rc = eng.get_rollout_config(mode)
    pad, eos = eng.rollout.pad_id(), eng.rollout.eos_id()
    prompts = list(training_input["prompts"])
    out = eng.generate(prompts=prompts, micro_batch_size=self._rollout_micro_batch_size)
    L = rc.max_tokens_to_generate
    comp = np.stack([common.pad_to_length(np.asarray(t), L, pad)[:L] for t in out.tokens]).astype(np.int64)
    prompt_ids = torch.from_numpy(np.asarray(out.left_padded_prompt_tokens)).long()
    completion_ids = torch.from_numpy(comp)
    B = completion_ids.shape[0]
    prompt_mask = (prompt_ids != pad).int()
    cmask = completion_ids != pad
    cm = cmask.float()
    eos_idx = common.build_positions_from_mask(cmask).max(dim=-1).values
    ref_lp = None
    if cfg.beta != 0.0:
      ref_lp = eng.get_ref_per_token_logps(prompt_ids, completion_ids, pad, eos,
                                           micro_batch_size=self._compute_logps_micro_batch_size).cpu()
    old_lp = eng.get_old_per_token_logps(prompt_ids, completion_ids,
                                         micro_batch_size=self._compute_logps_micro_batch_size).cpu()
    values = eng.get_values(prompt_ids, completion_ids, pad, eos).cpu().float()
    values = values[:, -L - 1:-1] * cm
    extra = {k: v for k, v in training_input.items() if k != "prompts"}
    if self._use_reward_model:
      scores = eng.get_rewards(prompt_ids, completion_ids, pad, eos).cpu().float()[:, -L:]
      last = scores[torch.arange(B), eos_idx]
    else:
      last = torch.as_tensor(self._compute_rewards(prompts=prompts, completions=out.text, mode=mode, **extra),
                             dtype=torch.float32)
    rewards = torch.zeros(B, L)
    rewards[torch.arange(B), eos_idx] += last
    kl = None
    if cfg.beta != 0.0:
      kl = common.compute_kl_divergence(old_lp, ref_lp, method=cfg.kl_method, clamp_value=cfg.kl_clamp_value) * cm
      rewards = rewards - cfg.beta * kl
    adv, ret = function_registry.get_advantage_estimator(cfg.advantage_estimator)(
        rewards=rewards, values=values, completion_mask=cm, gamma=cfg.gamma, gae_lambda=cfg.gae_lambda)
    ln = last.numpy()
    sr = rewards.sum(-1).numpy()
    eng.buffer_metrics({"rewards/score/mean": (ln.mean(), np.mean), "rewards/score/max": (ln.max(), np.max),
                        "rewards/score/min": (ln.min(), np.min), "rewards/reward/mean": (sr.mean(), np.mean),
                        "rewards/reward/max": (sr.max(), np.max), "rewards/reward/min": (sr.min(), np.min)}, mode=mode)
    if kl is not None:
      eng.buffer_metrics({"rewards/reward_kl_penalty": (float(masked_mean(kl, cm, axis=-1).mean()), np.mean)},
                         mode=mode)
    lens = cmask.sum(-1).numpy()
    eng.buffer_metrics({"generation/completions/mean_length": (lens.mean(), np.mean),
                        "generation/completions/max_length": (lens.max(), np.max),
                        "generation/completions/min_length": (lens.min(), np.min)}, mode=mode)
    inv = ~cmask.numpy()
    for name, arr in (("advantages", adv), ("advantages/returns", ret), ("advantages/old_values", values)):
      ma = np.ma.masked_array(arr.numpy(), mask=inv)
      eng.buffer_metrics({f"{name}/mean": (float(ma.mean()), np.mean), f"{name}/max": (float(ma.max()), np.max),
                          f"{name}/min": (float(ma.min()), np.min)}, mode=mode)
    for fn in self.metric_fns:
      eng.buffer_metrics(fn(prompts=prompts, completions=out.text, advantages=adv, rewards=ln, **extra), mode=mode)
    return TrainExample(prompt_ids=prompt_ids, prompt_mask=prompt_mask, completion_ids=completion_ids,
                        completion_mask=cmask, ref_per_token_logps=ref_lp, advantages=adv, returns=ret,
                        old_per_token_logps=old_lp, old_values=values)

  def _compute_trajectory_ids(self, example: TrainingInputT, steps: int) -> List[str]:
    bs = len(example["prompts"]) // self._num_generations()
    return np.arange(steps * bs, steps * bs + bs).astype(str).tolist()

  def _num_iterations(self) -> int:
    return self.algo_config.num_iterations

  def _num_generations(self) -> int:
    return 1


PpoConfig = PPOConfig
PpoLearner = PPOLearner
