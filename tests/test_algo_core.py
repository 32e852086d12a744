"""Policy and value losses of `rl/algo_core.py` against hand-computed values, with a stand-in model whose per-token
log-probs are dictated by the test: ratio clipping on both sides, dual clip for negative advantages, KL terms,
sampler importance weights, GSPO's sequence-level ratio, entropy bonus, value clipping; and the masked statistics."""
import math
import types

import numpy as np
import pytest
import torch

from tunix_b200.rl import algo_core, common


class DictatedPolicy(torch.nn.Module):
  """Logits such that log_softmax gives `token_logps[b][t]` to the token that follows position t."""

  def __init__(self, token_logps, vocab=6):
    super().__init__()
    self.token_logps, self.vocab = token_logps, vocab
    self.w = torch.nn.Parameter(torch.zeros(1))

  def forward(self, ids, positions=None, cache=None, attention_mask=None, **kw):
    rows, L = ids.shape
    logits = torch.full((rows, L, self.vocab), -40.0)
    for b in range(rows):
      for t in range(L - 1):
        lp = float(self.token_logps[b][t])
        target = int(ids[b, t + 1])
        logits[b, t, target] = lp
        logits[b, t, (target + 1) % self.vocab] = math.log(max(1.0 - math.exp(lp), 1e-12))
    return logits + 0.0 * self.w, None


def batch(new_logps, old_logps, advantages, ref=None, mask=None, **extra):
  """One prompt token, then the completion; `new_logps[b]` are the policy's log-probs of the completion tokens."""
  B, C = len(new_logps), len(new_logps[0])
  completion = torch.tensor([[1 + (k % 4) for k in range(C)]] * B)
  ex = common.TrainExample(
      prompt_ids=torch.full((B, 1), 5), prompt_mask=torch.ones(B, 1, dtype=torch.int32), completion_ids=completion,
      completion_mask=torch.ones(B, C, dtype=torch.int32) if mask is None else torch.tensor(mask, dtype=torch.int32),
      advantages=torch.tensor(advantages, dtype=torch.float32),
      ref_per_token_logps=None if ref is None else torch.tensor(ref, dtype=torch.float32),
      old_per_token_logps=None if old_logps is None else torch.tensor(old_logps, dtype=torch.float32), **extra)
  return DictatedPolicy(new_logps), ex


def grpo_cfg(**kw):
  base = dict(beta=0.0, epsilon=0.2, epsilon_high=None, epsilon_c=None, loss_algo="grpo", loss_agg_mode="token-mean",
              kl_loss_mode="low_var_kl", kl_clamp_value=None, temperature=1.0)
  base.update(kw)
  return types.SimpleNamespace(**base)


def val(x):
  return float(x.compute()) if hasattr(x, "compute") else float(x)


L = math.log


# ---- masked statistics ----------------------------------------------------------------------------------
def test_masked_statistics():
  x = torch.tensor([[1.0, 2.0, 30.0], [4.0, 50.0, 60.0]])
  m = torch.tensor([[1, 1, 0], [1, 0, 0]])
  assert float(algo_core.masked_mean(x, m)) == pytest.approx(7 / 3, rel=1e-6)
  assert algo_core.masked_mean(x, m, axis=1).tolist() == pytest.approx([1.5, 4.0], rel=1e-6)
  assert float(algo_core.masked_var(x, m)) == pytest.approx(np.var([1, 2, 4], ddof=1), rel=1e-5)      # Bessel
  w = algo_core.masked_whiten(x, m)
  kept = w[m.bool()]
  assert float(kept.mean()) == pytest.approx(0.0, abs=1e-5) and float(kept.var(unbiased=True)) == pytest.approx(1.0, rel=1e-4)


# ---- GRPO ---------------------------------------------------------------------------------------------------
def test_grpo_ratio_clipping_on_both_sides():
  # ratios 1.5 (A > 0: clipped to 1.2), 0.5 (A > 0: not clipped, the pessimistic branch), 0.5 (A < 0: clipped to 0.8)
  new = [[L(0.3), L(0.1)], [L(0.1), L(0.2)]]
  old = [[L(0.2), L(0.2)], [L(0.2), L(0.2)]]
  m, ex = batch(new, old, [2.0, -1.0])
  out = algo_core.grpo_loss_fn(m, ex, grpo_cfg(), 0, 0)
  per_token = [-2.0 * 1.2, -2.0 * 0.5, 1.0 * 0.8, 1.0 * 1.0]
  assert val(out.primary_loss) == pytest.approx(sum(per_token) / 4, rel=1e-4)
  aux = out.aux_metrics
  assert val(aux["pg_clipfrac"]) == pytest.approx(2 / 4) and val(aux["reduced_pg_loss"]) == pytest.approx(val(out.primary_loss), rel=1e-5)
  assert val(aux["is_ratio/max"]) == pytest.approx(1.5, rel=1e-4) and val(aux["is_ratio/min"]) == pytest.approx(0.5, rel=1e-4)
  assert val(aux["ppo_kl"]) == pytest.approx(-(L(1.5) + 2 * L(0.5) + 0.0) / 4, rel=1e-4)
  assert val(aux["advantage/abs_mean"]) == pytest.approx(1.5) and val(aux["advantage/nonzero_frac"]) == 1.0
  asym = algo_core.grpo_loss_fn(m, ex, grpo_cfg(epsilon_high=0.4), 0, 0)                      # DAPO's wider upper side
  assert val(asym.primary_loss) == pytest.approx((-2.0 * 1.4 - 1.0 + 0.8 + 1.0) / 4, rel=1e-4)


def test_grpo_dual_clip_bounds_the_loss_of_bad_actions_that_became_likelier():
  new, old = [[L(0.8)]], [[L(0.1)]]                                       # ratio 8 on a negative advantage
  m, ex = batch(new, old, [-1.0])
  plain = algo_core.grpo_loss_fn(m, ex, grpo_cfg(), 0, 0)
  assert val(plain.primary_loss) == pytest.approx(8.0, rel=1e-4)
  capped = algo_core.grpo_loss_fn(m, ex, grpo_cfg(epsilon_c=3.0), 0, 0)
  assert val(capped.primary_loss) == pytest.approx(3.0, rel=1e-4) and val(capped.aux_metrics["pg_clipfrac_lower"]) == 1.0
  m, ex = batch(new, old, [1.0])                                           # positive advantages are never dual-clipped
  assert val(algo_core.grpo_loss_fn(m, ex, grpo_cfg(epsilon_c=3.0), 0, 0).primary_loss) == pytest.approx(-1.2, rel=1e-4)


def test_grpo_without_old_logps_is_on_policy_and_the_gradient_is_the_advantage():
  m, ex = batch([[L(0.3), L(0.4)]], None, [2.0])
  out = algo_core.grpo_loss_fn(m, ex, grpo_cfg(), 0, 0)
  assert val(out.primary_loss) == pytest.approx(-2.0, rel=1e-5) and val(out.aux_metrics["pg_clipfrac"]) == 0.0


def test_grpo_kl_term_masks_and_modes():
  new, old, ref = [[L(0.3), L(0.3)]], [[L(0.3), L(0.3)]], [[L(0.2), L(0.6)]]
  m, ex = batch(new, old, [0.0], ref=ref, mask=[[1, 0]])                  # the second token is masked out
  out = algo_core.grpo_loss_fn(m, ex, grpo_cfg(beta=0.5, kl_loss_mode="low_var_kl"), 0, 0)
  d = L(0.2) - L(0.3)
  kl = math.exp(d) - d - 1
  assert val(out.aux_metrics["kl"]) == pytest.approx(kl, rel=1e-4) and val(out.primary_loss) == pytest.approx(0.5 * kl, rel=1e-4)
  straight = algo_core.grpo_loss_fn(m, ex, grpo_cfg(beta=1.0, kl_loss_mode="kl", kl_clamp_value=0.1), 0, 0)
  assert val(straight.primary_loss) == pytest.approx(0.1, rel=1e-4)                          # L(0.3) - L(0.2) = 0.405, clamped
  m2, ex2 = batch(new, old, [0.0])
  with pytest.raises(ValueError, match="requires ref_per_token_logps"):
    algo_core.grpo_loss_fn(m2, ex2, grpo_cfg(beta=0.1), 0, 0)
  assert val(algo_core.grpo_loss_fn(m2, ex2, grpo_cfg(beta=None), 0, 0).aux_metrics["kl"]) == 0.0


def test_grpo_sampler_weights_scale_tokens_and_aggregation_modes_differ():
  new = [[L(0.2), L(0.2)], [L(0.2), L(0.2)]]
  m, ex = batch(new, new, [1.0, 3.0], mask=[[1, 1], [1, 0]], sampler_is_weights=torch.tensor([[1.0, 0.5], [2.0, 9.0]]))
  out = algo_core.grpo_loss_fn(m, ex, grpo_cfg(), 0, 0)
  assert val(out.primary_loss) == pytest.approx(-(1.0 + 0.5 + 6.0) / 3, rel=1e-4)
  assert val(out.aux_metrics["sampler_is/weight_mean"]) == pytest.approx(3.5 / 3, rel=1e-5)
  assert val(out.aux_metrics["sampler_is/weight_min"]) == 0.5
  per_seq = algo_core.grpo_loss_fn(m, ex, grpo_cfg(loss_agg_mode="sequence-mean-token-mean"), 0, 0)
  assert val(per_seq.primary_loss) == pytest.approx(-((1.0 + 0.5) / 2 + 6.0) / 2, rel=1e-4)


def test_gspo_token_uses_the_sequence_mean_ratio_for_every_token():
  new, old = [[L(0.4), L(0.1)]], [[L(0.2), L(0.2)]]                        # token ratios 2 and 0.5: sequence ratio 1
  m, ex = batch(new, old, [1.0])
  token_level = algo_core.grpo_loss_fn(m, ex, grpo_cfg(), 0, 0)
  assert val(token_level.primary_loss) == pytest.approx(-(1.2 + 0.5) / 2, rel=1e-4)
  seq_level = algo_core.grpo_loss_fn(m, ex, grpo_cfg(loss_algo="gspo-token"), 0, 0)
  assert val(seq_level.primary_loss) == pytest.approx(-1.0, rel=1e-4) and val(seq_level.aux_metrics["pg_clipfrac"]) == 0.0
  seq_level.primary_loss.unreduced_sum.backward()                            # the gradient still flows per token
  assert m.w.grad is not None


def test_token_level_advantages_are_used_as_given():
  new = [[L(0.2), L(0.2), L(0.2)]]
  m, ex = batch(new, new, [[1.0, -2.0, 0.0]])
  out = algo_core.grpo_loss_fn(m, ex, grpo_cfg(), 0, 0)
  assert val(out.primary_loss) == pytest.approx((-1.0 + 2.0 + 0.0) / 3, rel=1e-4)
  assert val(out.aux_metrics["advantage/nonzero_frac"]) == pytest.approx(2 / 3, rel=1e-5)


# ---- PPO ----------------------------------------------------------------------------------------------------
def ppo_cfg(**kw):
  base = dict(epsilon_low=0.2, epsilon_high=0.3, epsilon_c=None, entropy_coef=None, kl_coef=0.0, kl_clamp_value=None)
  base.update(kw)
  return types.SimpleNamespace(**base)


def test_ppo_policy_loss_clip_dual_clip_entropy_and_kl():
  new, old = [[L(0.3), L(0.05)]], [[L(0.2), L(0.2)]]                       # ratios 1.5 and 0.25
  m, ex = batch(new, old, [[1.0, -1.0]], ref=[[L(0.3), L(0.1)]])
  out = algo_core.ppo_policy_loss_fn(m, ex, ppo_cfg(), 0, 0)
  assert val(out.primary_loss) == pytest.approx((-1.3 + 0.8) / 2, rel=1e-4)   # upper side at 1 + 0.3, lower at 1 - 0.2
  assert val(out.aux_metrics["pg_clipfrac"]) == 1.0
  with_kl = algo_core.ppo_policy_loss_fn(m, ex, ppo_cfg(kl_coef=2.0), 0, 0)
  kl = (0.0 + (L(0.05) - L(0.1))) / 2
  assert val(with_kl.aux_metrics["kl"]) == pytest.approx(kl, rel=1e-4)
  assert val(with_kl.primary_loss) == pytest.approx((-1.3 + 0.8) / 2 + 2.0 * kl, rel=1e-4)
  with_entropy = algo_core.ppo_policy_loss_fn(m, ex, ppo_cfg(entropy_coef=0.5), 0, 0)
  ent = val(with_entropy.aux_metrics["loss/entropy"])
  h = lambda p: -(p * L(p) + (1 - p) * L(1 - p))                             # the stand-in puts the rest on one token
  assert ent == pytest.approx((h(0.3) + h(0.05)) / 2, rel=1e-3)
  assert val(with_entropy.primary_loss) == pytest.approx((-1.3 + 0.8) / 2 - 0.5 * ent, rel=1e-4)
  m2, ex2 = batch([[L(0.9)]], [[L(0.1)]], [[-1.0]])
  assert val(algo_core.ppo_policy_loss_fn(m2, ex2, ppo_cfg(), 0, 0).primary_loss) == pytest.approx(9.0, rel=1e-4)
  dual = algo_core.ppo_policy_loss_fn(m2, ex2, ppo_cfg(epsilon_c=2.0), 0, 0)
  assert val(dual.primary_loss) == pytest.approx(2.0, rel=1e-4) and val(dual.aux_metrics["pg_clipfrac_lower"]) == 1.0


def test_ppo_value_loss_clips_around_the_old_values():
  class Critic(torch.nn.Module):
    def __init__(self, values):
      super().__init__()
      self.values, self.w = values, torch.nn.Parameter(torch.zeros(1))
    def forward(self, ids, positions=None, cache=None, attention_mask=None, **kw):
      return self.values[..., None] + 0.0 * self.w, None
  # positions: [prompt, c0, c1]; the value of a completion token is read at the position before it
  critic = Critic(torch.tensor([[1.0, 3.0, 99.0]]))
  _, ex = batch([[0.0, 0.0]], None, [0.0])
  holder = types.SimpleNamespace(prompt_ids=ex.prompt_ids, completion_ids=ex.completion_ids,
                                 completion_mask=ex.completion_mask, old_values=torch.tensor([[0.5, 1.0]]),
                                 returns=torch.tensor([[2.0, 2.0]]), segment_ids=None, segment_positions=None)
  out = algo_core.ppo_value_loss_fn(critic, holder, clip_range_value=0.5, pad_id=0, eos_id=0)
  # predictions 1.0 and 3.0; clipped to [0.0, 1.0] -> 1.0 and [0.5, 1.5] -> 1.5
  v1 = [(1.0 - 2.0) ** 2, (3.0 - 2.0) ** 2]
  v2 = [(1.0 - 2.0) ** 2, (1.5 - 2.0) ** 2]
  assert val(out.primary_loss) == pytest.approx(0.5 * (max(v1[0], v2[0]) + max(v1[1], v2[1])) / 2, rel=1e-5)
  assert val(out.aux_metrics["vpred_mean"]) == 2.0 and val(out.aux_metrics["return_mean"]) == 2.0
  assert val(out.aux_metrics["vf_clipfrac"]) == 0.0                            # clipping never made the error larger here
  unclipped = algo_core.ppo_value_loss_fn(critic, holder, clip_range_value=None, pad_id=0, eos_id=0)
  assert val(unclipped.primary_loss) == pytest.approx(0.5 * (1.0 + 1.0) / 2, rel=1e-5)
