"""DPO / ORPO trainers on CPU: loss values against a direct restatement, training progress,
string and tokenised inputs."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from tunix_b200 import optim
from tunix_b200.models.transformer import ModelConfig, Transformer
from tunix_b200.sft.dpo import dpo_trainer as dpo


class Tok:
  def encode(self, s, **k): return [3 + (ord(c) % 60) for c in s]
  def decode(self, ids, **k): return "".join(chr(32 + int(i)) for i in ids)
  def bos_id(self): return 1
  def eos_id(self): return 2
  def pad_id(self): return 0


def model(seed=0):
  cfg = ModelConfig(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=4, head_dim=8, num_kv_heads=2)
  return Transformer(cfg).init_weights(seed=seed, scale=0.2)


def data(n=2):
  return [dpo.DataInput(prompts=["what is up", "tell me"], chosen_responses=["good answer", "fine"],
                        rejected_responses=["bad", "terrible reply"]) for _ in range(n)]


def cfg(**kw):
  kw.setdefault("eval_every_n_steps", 100)
  kw.setdefault("pbar_description", None)
  kw.setdefault("max_prompt_length", 12)
  kw.setdefault("max_response_length", 16)
  return dpo.DPOTrainingConfig(**kw)


def test_dpo_loss_matches_restatement_and_trains():
  m, ref = model(0), model(0)
  tr = dpo.DPOTrainer(m, ref, optim.adamw(5e-3), cfg(max_steps=6, beta=0.2, label_smoothing=0.1), tokenizer=Tok())
  ex = tr._prepare_inputs(data(1)[0])
  out = dpo.dpo_loss_fn(m, ex, beta=0.2, label_smoothing=0.1)
  # identical policy and reference: delta = 0 -> loss = log 2 per pair
  assert abs(out.primary_loss.compute().item() - np.log(2.0)) < 1e-5
  assert float(out.primary_loss.denominator) == 2.0
  tr.train(data(6))
  losses = tr.metrics_logger.get_metric_history("", "loss", "train")
  assert losses[-1] < losses[0]
  acc = tr.metrics_logger.get_metric_history("", "rewards/accuracy", "train")
  assert acc[-1] == 1.0
  assert tr.metrics_logger.metric_exists("", "rewards/margin", "train")


def test_dpo_direct_restatement_of_loss():
  torch.manual_seed(0)
  m, ref = model(1), model(2)
  tr = dpo.DPOTrainer(m, ref, optim.sgd(0.1), cfg(), tokenizer=Tok())
  ex = tr._prepare_inputs(data(1)[0])
  out = dpo.dpo_loss_fn(m, ex, beta=0.1)

  def seq_logp(mod):
    logits, _ = mod(ex.input_ids, ex.positions, None, ex.attention_mask)
    lp = torch.log_softmax(logits.float(), -1)[:, :-1].gather(-1, ex.input_ids[:, 1:, None])[..., 0]
    k = ex.logits_to_keep
    return (lp[:, -k:] * ex.completion_mask).sum(-1)
  with torch.no_grad():
    pi, rf = seq_logp(m), seq_logp(ref)
  d = (pi[:2] - rf[:2]) - (pi[2:] - rf[2:])
  want = -F.logsigmoid(0.1 * d).mean()
  torch.testing.assert_close(out.primary_loss.compute().detach(), want, rtol=1e-4, atol=1e-5)


def test_orpo_trains_without_reference_and_tokenised_input():
  m = model(3)
  tr = dpo.ORPOTrainer(m, None, optim.adamw(5e-3), cfg(algorithm="orpo", max_steps=4), tokenizer=Tok())
  rec = dpo.process_dpo_record({"prompts": ["a b", "c"], "chosen_responses": ["yes", "ok"],
                                "rejected_responses": ["no", "nah"]}, tr.tokenizer, 8, 8)
  assert rec.prompt_ids.shape == (2, 8) and rec.prompt_mask[0, 0] == 0 and rec.chosen_mask[0, -1] == 0
  batch = {f.name: getattr(rec, f.name) for f in __import__("dataclasses").fields(rec)}
  tr.train([batch] * 4)
  assert tr.train_steps == 4
  lg = tr.metrics_logger
  assert lg.metric_exists("", "odds_ratio", "train") and lg.metric_exists("", "sft_loss", "train")
  l = lg.get_metric_history("", "loss", "train")
  assert l[-1] < l[0]
  with pytest.raises(ValueError):
    tr._prepare_inputs({"foo": 1})


def test_reference_with_adapters_off_shares_the_backbone():
  """DPO with a LoRA policy and `ReferenceWithAdaptersOff`: at zero adapter output policy == reference, so the
  first loss is log 2; adapters train, the backbone does not, and the reference ignores the adapters."""
  import numpy as np
  from tunix_b200 import optim
  from tunix_b200.models import lora
  from tunix_b200.models.transformer import ModelConfig, Transformer
  from tunix_b200.sft.dpo import dpo_trainer as dpo
  torch.manual_seed(0)
  cfg = ModelConfig(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=4, head_dim=8, num_kv_heads=2)
  model = Transformer(cfg).init_weights(seed=0, scale=0.3)
  lora.apply_lora_to_model(model, rank=4, alpha=8.0)
  ref = dpo.ReferenceWithAdaptersOff(model)
  assert not list(ref.parameters())
  g = torch.Generator().manual_seed(1)
  ti = dpo.TrainingInput(prompt_ids=torch.randint(1, 64, (4, 6), generator=g), prompt_mask=torch.ones(4, 6),
                         chosen_ids=torch.randint(1, 64, (4, 5), generator=g), chosen_mask=torch.ones(4, 5),
                         rejected_ids=torch.randint(1, 64, (4, 5), generator=g), rejected_mask=torch.ones(4, 5))
  tc = dpo.DPOTrainingConfig(eval_every_n_steps=100, max_steps=6, pbar_description=None, beta=0.5)
  tr = dpo.DPOTrainer(model, ref, optim.adamw(5e-2), tc)
  base = {n: p.clone() for n, p in model.named_parameters() if "lora" not in n}
  tr.train([ti] * 6)
  losses = tr.metrics_logger.get_metric_history("", "loss", "train")
  np.testing.assert_allclose(losses[0], np.log(2.0), rtol=1e-4)
  assert losses[-1] < losses[0]
  for n, p in model.named_parameters():
    if "lora" not in n:
      assert torch.equal(p, base[n])
  toks = torch.randint(1, 64, (2, 7), generator=g)
  with_adapters, _ = model(toks, None, None, None)
  without, _ = ref(toks, None, None, None)
  assert not torch.allclose(with_adapters, without)
  assert all(v != 0 for m in model.modules() if hasattr(m, "lora_scale") for v in m.lora_scale.values())
