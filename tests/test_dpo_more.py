"""DPO / ORPO beyond the basics: input preparation from strings and token arrays, the loss against hand-computed
values (label smoothing, reference terms, ORPO with prompt loss and length-averaging), logged metrics, and
configuration errors."""
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from tunix_b200 import optim
from tunix_b200.sft.dpo import dpo_trainer as dpo
from tunix_b200.sft.utils import LossOutput
from tests.test_dpo import Tok, cfg, data, model


# ---- input preparation ------------------------------------------------------------------------------
def test_records_are_tokenised_with_prompts_left_padded_and_responses_right_padded():
  tok = dpo.tokenizer_adapter.TokenizerAdapter(Tok())
  rec = {"prompts": ["ab", "abcdef"], "chosen_responses": ["xyz", "x"], "rejected_responses": ["q", "qrstu"]}
  ti = dpo.process_dpo_record(rec, tok, max_prompt_length=5, max_response_length=4)
  assert ti.prompt_ids.shape == (2, 5) and ti.chosen_ids.shape == (2, 4) and ti.rejected_ids.shape == (2, 4)
  assert ti.prompt_mask.tolist() == [[0, 0, 1, 1, 1], [1, 1, 1, 1, 1]]            # BOS + text, long prompts cut to length
  assert ti.prompt_ids[0, 2].item() == 1                                            # the BOS survives the padding
  assert ti.chosen_mask.tolist() == [[1, 1, 1, 1], [1, 1, 0, 0]] and ti.rejected_mask.tolist() == [[1, 1, 0, 0], [1, 1, 1, 1]]
  single = dpo.process_dpo_record({"prompts": "ab", "chosen_responses": "x", "rejected_responses": "y"}, tok, 4, 3)
  assert single.prompt_ids.shape == (4,) and single.chosen_ids.shape == (3,)        # one record: no batch axis
  with pytest.raises(ValueError, match="either tokenized fields"):
    dpo._preprocess_dict({"prompts": ["a"]})
  assert isinstance(dpo._preprocess_dict(rec), dpo.DataInput)
  as_dict = {f: getattr(ti, f) for f in ("prompt_ids", "prompt_mask", "chosen_ids", "chosen_mask", "rejected_ids", "rejected_mask")}
  assert isinstance(dpo._preprocess_dict(as_dict), dpo.TrainingInput)


def test_the_train_example_stacks_chosen_over_rejected_and_carries_reference_logps():
  policy, ref = model(0), model(1)
  tr = dpo.DPOTrainer(policy, ref, optim.adamw(1e-3), cfg(), tokenizer=Tok())
  ex = tr._prepare_inputs(data(1)[0])
  B = 2
  assert ex.input_ids.shape == (2 * B, 12 + 16) and ex.logits_to_keep == 16 and ex.completion_mask.shape == (2 * B, 16)
  assert torch.equal(ex.input_ids[:B, :12], ex.input_ids[B:, :12])                  # the same prompts under both halves
  assert not torch.equal(ex.input_ids[:B, 12:], ex.input_ids[B:, 12:])
  assert ex.ref_chosen_logps.shape == (B,) and not ex.ref_chosen_logps.requires_grad
  want_c, want_r, _ = dpo.compute_logps(ref, ex.input_ids, ex.positions, ex.attention_mask, 16, ex.completion_mask)
  torch.testing.assert_close(ex.ref_chosen_logps, want_c)
  torch.testing.assert_close(ex.ref_rejected_logps, want_r)
  assert tr._prepare_inputs(ex) is ex                                                # already prepared: passes through
  no_ref = dpo.DPOTrainer(model(0), None, optim.adamw(1e-3), cfg(algorithm="orpo"), tokenizer=Tok())
  assert no_ref._prepare_inputs(data(1)[0]).ref_chosen_logps is None
  tr.close(); no_ref.close()


def test_string_inputs_need_a_tokenizer_and_lengths():
  tr = dpo.DPOTrainer(model(), None, optim.adamw(1e-3), cfg(algorithm="orpo"))
  with pytest.raises(ValueError, match="Tokenizer must be provided"):
    tr._prepare_inputs(data(1)[0])
  tr.close()
  tr = dpo.DPOTrainer(model(), None, optim.adamw(1e-3), cfg(algorithm="orpo", max_prompt_length=None), tokenizer=Tok())
  with pytest.raises(ValueError, match="max_prompt_length and max_response_length must be provided"):
    tr._prepare_inputs(data(1)[0])
  tr.close()


# ---- the loss by hand ---------------------------------------------------------------------------------
class FixedLogps(torch.nn.Module):
  """A "model" whose per-token log-probs are what the test says: logits are chosen so that log_softmax gives them."""

  def __init__(self, token_logps):
    super().__init__()
    self.token_logps = token_logps                     # [rows, L - 1]: log-prob of token t+1 at position t
    self.w = torch.nn.Parameter(torch.zeros(1))

  def forward(self, ids, positions=None, cache=None, attention_mask=None, **kw):
    rows, L = ids.shape
    V = 8
    logits = torch.full((rows, L, V), -30.0)
    for b in range(rows):
      for t in range(L - 1):
        lp = float(self.token_logps[b][t])
        target = int(ids[b, t + 1])
        # two-way split: the target gets lp, one other token takes the rest of the mass
        other = (target + 1) % V
        logits[b, t, target] = lp
        logits[b, t, other] = math.log(max(1.0 - math.exp(lp), 1e-12))
    return logits + 0.0 * self.w, None


def example(lps_chosen, lps_rejected, ref=None, prompt_len=1):
  n = len(lps_chosen)
  ids = torch.tensor([[1] * prompt_len + [2 + (k % 5) for k in range(n)]] * 2)
  comp_mask = torch.ones(2, n, dtype=torch.int32)
  full = torch.ones(2, prompt_len + n, dtype=torch.int32)
  pad = [math.log(0.5)] * (prompt_len - 1)
  token_logps = [pad + list(lps_chosen), pad + list(lps_rejected)]
  ex = dpo.TrainExample(input_ids=ids, positions=torch.arange(prompt_len + n).expand(2, -1), attention_mask=None,
                        ref_chosen_logps=None if ref is None else torch.tensor([ref[0]]),
                        ref_rejected_logps=None if ref is None else torch.tensor([ref[1]]),
                        completion_mask=comp_mask, logits_to_keep=n, full_mask=full)
  return FixedLogps(token_logps), ex


def test_dpo_loss_by_hand_with_reference_and_label_smoothing():
  chosen, rejected = [math.log(0.5), math.log(0.4)], [math.log(0.2), math.log(0.1)]
  m, ex = example(chosen, rejected, ref=(-2.0, -3.0))
  c, r = sum(chosen), sum(rejected)
  delta = (c + 2.0) - (r + 3.0)
  for beta, eps in ((0.1, 0.0), (0.5, 0.2)):
    out = dpo.dpo_loss_fn(m, ex, beta=beta, label_smoothing=eps)
    assert isinstance(out, LossOutput)
    want = -(F.logsigmoid(torch.tensor(beta * delta)) * (1 - eps) + F.logsigmoid(torch.tensor(-beta * delta)) * eps)
    assert float(out.primary_loss.compute()) == pytest.approx(float(want), rel=1e-4)
    aux = {k: float(v.compute()) for k, v in out.aux_metrics.items()}
    assert aux["rewards/chosen"] == pytest.approx(beta * (c + 2.0), rel=1e-4)
    assert aux["rewards/margin"] == pytest.approx(beta * delta, rel=1e-4) and aux["rewards/accuracy"] == 1.0
    assert aux["log_probs/chosen"] == pytest.approx(c, rel=1e-4) and aux["log_probs/rejected"] == pytest.approx(r, rel=1e-4)
  m, ex = example(chosen, rejected)                              # without a reference the raw log-probs are compared
  out = dpo.dpo_loss_fn(m, ex, beta=1.0)
  assert float(out.primary_loss.compute()) == pytest.approx(float(-F.logsigmoid(torch.tensor(c - r))), rel=1e-4)


@pytest.mark.parametrize("average, prompt_loss", [(False, False), (True, False), (True, True), (False, True)])
def test_orpo_loss_by_hand(average, prompt_loss):
  chosen, rejected = [math.log(0.6), math.log(0.5), math.log(0.7)], [math.log(0.3), math.log(0.2), math.log(0.4)]
  m, ex = example(chosen, rejected, prompt_len=3)
  lam = 0.25
  out = dpo.dpo_loss_fn(m, ex, algorithm="orpo", lambda_orpo=lam, average_log_prob_orpo=average,
                        enable_prompt_loss_orpo=prompt_loss)
  c, r = sum(chosen), sum(rejected)
  if average:
    c, r = c / 3, r / 3
  if prompt_loss:
    full = 2 * math.log(0.5) + sum(chosen)                       # prompt tokens after the first, then the answer
    sft = -full / 5 if average else -full
  else:
    sft = -c
  log_odds = (c - r) - (math.log1p(-math.exp(c)) - math.log1p(-math.exp(r)))
  or_loss = -float(F.logsigmoid(torch.tensor(log_odds)))
  aux = {k: float(v.compute()) for k, v in out.aux_metrics.items()}
  assert aux["sft_loss"] == pytest.approx(sft, rel=1e-4) and aux["or_loss"] == pytest.approx(or_loss, rel=1e-4)
  assert float(out.primary_loss.compute()) == pytest.approx(sft + lam * or_loss, rel=1e-4)
  assert aux["odds_ratio"] == pytest.approx(math.exp(log_odds), rel=1e-4) and aux["rewards/accuracy"] == 1.0


# ---- training loop ------------------------------------------------------------------------------------
def test_training_logs_the_preference_metrics_and_raises_the_margin():
  tr = dpo.DPOTrainer(model(0), model(0), optim.adamw(5e-3), cfg(gradient_accumulation_steps=2), tokenizer=Tok())
  tr.train(data(8))
  lg = tr.metrics_logger
  for name in ("rewards/chosen", "rewards/rejected", "rewards/margin", "rewards/accuracy", "log_probs/chosen",
               "log_probs/rejected"):
    assert len(lg.get_metric_history("", name, "train")) == 4, name
  margins = lg.get_metric_history("", "rewards/margin", "train")
  assert margins[0] == pytest.approx(0.0, abs=1e-5) and margins[-1] > margins[0]   # policy = reference at the start
  assert not lg.metric_exists("", "odds_ratio", "train")
  orpo = dpo.ORPOTrainer(model(0), None, optim.adamw(5e-3), dpo.ORPOTrainingConfig(
      algorithm="orpo", eval_every_n_steps=100, pbar_description=None, max_prompt_length=12, max_response_length=16),
      tokenizer=Tok())
  orpo.train(data(3), eval_ds=data(1))
  assert len(orpo.metrics_logger.get_metric_history("", "odds_ratio", "train")) == 3
  assert orpo.metrics_logger.metric_exists("", "rewards/margin", "eval")


def test_tokenised_and_dict_inputs_train_like_string_inputs():
  strings = data(2)
  tok = dpo.tokenizer_adapter.TokenizerAdapter(Tok())
  tokenised = [dpo.process_dpo_record({"prompts": d.prompts, "chosen_responses": d.chosen_responses,
                                       "rejected_responses": d.rejected_responses}, tok, 12, 16) for d in strings]
  as_dicts = [{"prompts": d.prompts, "chosen_responses": d.chosen_responses, "rejected_responses": d.rejected_responses}
              for d in strings]
  finals = []
  for stream, tokenizer in ((strings, Tok()), (tokenised, None), (as_dicts, Tok())):
    m = model(3)
    dpo.DPOTrainer(m, model(3), optim.adamw(1e-2), cfg(), tokenizer=tokenizer).train(stream)
    finals.append({n: p.detach().clone() for n, p in m.named_parameters()})
  for other in finals[1:]:
    for n in finals[0]:
      torch.testing.assert_close(finals[0][n], other[n], msg=n)
