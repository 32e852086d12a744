"""DPO (https://arxiv.org/abs/2305.18290) and ORPO (https://arxiv.org/abs/2403.07691) trainers
(tunix/sft/dpo/dpo_trainer.py:42-798).

Inputs are raw strings (`DataInput`, tokenised here: prompts left-padded, responses
right-padded) or token ids (`TrainingInput`). Chosen and rejected rows are concatenated on the
batch axis so one forward pass scores both. For DPO the frozen reference log-probabilities are
computed in `_prepare_inputs`, outside the differentiated step.

DPO loss: `-[log sigmoid(beta d)(1 - ls) + log sigmoid(-beta d) ls]` with
`d = (pi_c - ref_c) - (pi_r - ref_r)` over summed completion log-probs; denominator = #pairs.
ORPO: SFT NLL (length-averaged, prompt + completion by default) + lambda * odds-ratio loss with
`log_odds = (c - r) - (log1p(-e^c) - log1p(-e^r))`, log-probs clipped to <= -1e-7.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Union

import numpy as np
import torch
import torch.nn.functional as F

from ...common.configs import TrainingConfig
from ...generate import tokenizer_adapter
from ...rl import common
from .. import peft_trainer
from .. import utils as sft_utils

WeightedMetric = sft_utils.WeightedMetric


@dataclasses.dataclass(frozen=True)
class DataInput:
  """Raw-string training input."""
  prompts: List[str]
  chosen_responses: List[str]
  rejected_responses: List[str]
  images: Any = None


@dataclasses.dataclass(frozen=True)
class TrainingInput:
  """Tokenised input: prompts left-padded, responses right-padded."""
  prompt_ids: Any
  prompt_mask: Any
  chosen_ids: Any
  chosen_mask: Any
  rejected_ids: Any
  rejected_mask: Any
  images: Any = None


@dataclasses.dataclass(frozen=True)
class TrainExample:
  input_ids: torch.Tensor          # [2B, P + R]: chosen rows then rejected rows
  positions: torch.Tensor
  attention_mask: torch.Tensor
  ref_chosen_logps: Optional[torch.Tensor]
  ref_rejected_logps: Optional[torch.Tensor]
  completion_mask: torch.Tensor
  logits_to_keep: int
  images: Any = None
  full_mask: Optional[torch.Tensor] = None


class ReferenceWithAdaptersOff(torch.nn.Module):
  """The frozen reference of a LoRA policy: the same module with every adapter's scale set to zero for the
  duration of the call, so no second copy of the backbone is held."""

  def __init__(self, model: torch.nn.Module):
    super().__init__()
    object.__setattr__(self, "_policy", model)      # not registered: its parameters stay the policy's

  @property
  def config(self):
    return self._policy.config

  def forward(self, *args, **kwargs):
    saved = []
    for mod in self._policy.modules():
      sc = getattr(mod, "lora_scale", None)
      if isinstance(sc, dict) and sc:
        saved.append((mod, dict(sc)))
        for k in sc:
          sc[k] = 0.0
    try:
      with torch.no_grad():
        return self._policy(*args, **kwargs)
    finally:
      for mod, sc in saved:
        mod.lora_scale.update(sc)


@dataclasses.dataclass(kw_only=True)
class DPOTrainingConfig(TrainingConfig):
  algorithm: str = "dpo"            # "dpo" or "orpo"
  beta: float = 0.1                 # DPO only
  lambda_orpo: float = 0.1          # ORPO only
  label_smoothing: float = 0.0
  enable_prompt_loss_orpo: bool = True
  average_log_prob_orpo: bool = True
  max_prompt_length: Optional[int] = None
  max_response_length: Optional[int] = None


def compute_logps(model, input_ids, positions, attention_mask, logits_to_keep: int, completion_mask, images=None,
                  enable_prompt_loss_orpo: bool = False, full_mask=None):
  """-> (chosen_logps [B], rejected_logps [B], prompt+chosen logps [B] or None): summed log-probs."""
  cm = completion_mask.float()
  if enable_prompt_loss_orpo:
    tok = common.get_per_token_logps(model, input_ids, positions, attention_mask, input_ids.shape[1] - 1, images)
    comp = (tok[:, -cm.shape[-1]:] * cm).sum(-1)
    full = (tok * full_mask[:, 1:].float()).sum(-1)
    B = tok.shape[0] // 2
    return comp[:B], comp[B:], full[:B]
  tok = common.get_per_token_logps(model, input_ids, positions, attention_mask, logits_to_keep, images)
  s = (tok * cm).sum(-1)
  B = s.shape[0] // 2
  return s[:B], s[B:], None


def _wm(x, denom):
  return WeightedMetric(x, denom, min_denom=1.0)


def dpo_loss_fn(model, train_example: TrainExample, algorithm: str = "dpo", beta: float = 0.1,
                lambda_orpo: float = 0.1, label_smoothing: float = 0.0, enable_prompt_loss_orpo: bool = False,
                average_log_prob_orpo: bool = False) -> sft_utils.LossOutput:
  ex = train_example
  c, r, pc = compute_logps(model, ex.input_ids, ex.positions, ex.attention_mask, ex.logits_to_keep,
                           ex.completion_mask, ex.images, enable_prompt_loss_orpo, ex.full_mask)
  B = ex.completion_mask.shape[0] // 2
  denom = torch.tensor(float(B), device=c.device)
  if algorithm == "orpo":
    if average_log_prob_orpo:
      cm = ex.completion_mask.float()
      c = c / cm[:B].sum(-1).clamp(min=1.0)
      r = r / cm[B:].sum(-1).clamp(min=1.0)
    if enable_prompt_loss_orpo:
      sft = -pc / ex.full_mask[:B, 1:].float().sum(-1).clamp(min=1.0) if average_log_prob_orpo else -pc
    else:
      sft = -c
    c, r = torch.clamp(c, max=-1e-7), torch.clamp(r, max=-1e-7)
    log_odds = (c - r) - (torch.log1p(-torch.exp(c)) - torch.log1p(-torch.exp(r)))
    or_loss = -(F.logsigmoid(log_odds) * (1 - label_smoothing) + F.logsigmoid(-log_odds) * label_smoothing)
    total = sft + lambda_orpo * or_loss
    cr, rr = lambda_orpo * c, lambda_orpo * r
    aux = {"rewards/chosen": _wm(cr.sum().detach(), denom), "rewards/rejected": _wm(rr.sum().detach(), denom),
           "rewards/margin": _wm((cr - rr).sum().detach(), denom),
           "rewards/accuracy": _wm((cr > rr).float().sum(), denom),
           "log_probs/chosen": _wm(c.sum().detach(), denom), "log_probs/rejected": _wm(r.sum().detach(), denom),
           "odds_ratio": _wm(torch.exp(log_odds).sum().detach(), denom), "sft_loss": _wm(sft.sum().detach(), denom),
           "or_loss": _wm(or_loss.sum().detach(), denom)}
    return sft_utils.LossOutput(primary_loss=_wm(total.sum(), denom), aux_metrics=aux)
  clr = c - ex.ref_chosen_logps if ex.ref_chosen_logps is not None else c
  rlr = r - ex.ref_rejected_logps if ex.ref_rejected_logps is not None else r
  delta = clr - rlr
  losses = -(F.logsigmoid(beta * delta) * (1 - label_smoothing) + F.logsigmoid(-beta * delta) * label_smoothing)
  cr, rr = beta * clr, beta * rlr
  aux = {"rewards/chosen": _wm(cr.sum().detach(), denom), "rewards/rejected": _wm(rr.sum().detach(), denom),
         "rewards/margin": _wm((cr - rr).sum().detach(), denom), "rewards/accuracy": _wm((cr > rr).float().sum(), denom),
         "log_probs/chosen": _wm(c.sum().detach(), denom), "log_probs/rejected": _wm(r.sum().detach(), denom)}
  return sft_utils.LossOutput(primary_loss=_wm(losses.sum(), denom), aux_metrics=aux)


def _tokenize(s: str, tokenizer) -> np.ndarray:
  ids = list(tokenizer.encode(s))
  bos = [tokenizer.bos_id()] if tokenizer.bos_id() else []
  return np.array(tokenizer.dedup_bos_ids(bos + ids), dtype=np.int64)


def _generate_ids_and_masks(strings: List[str], tokenizer, max_length: int, left_pad: bool = True):
  pad = tokenizer.pad_id()
  ids = np.stack([common.pad_to_length(_tokenize(s, tokenizer)[:max_length], max_length, pad, left=left_pad, axis=-1)
                  for s in strings])
  return torch.from_numpy(ids), torch.from_numpy((ids != pad).astype(np.int32))


def _preprocess_dict(d: Dict[str, Any]) -> Union[DataInput, TrainingInput]:
  tok = [f.name for f in dataclasses.fields(TrainingInput)]
  raw = [f.name for f in dataclasses.fields(DataInput)]
  if all(f in d for f in tok if f != "images"):
    return TrainingInput(**{f: d.get(f) for f in tok})
  if all(f in d for f in raw if f != "images"):
    return DataInput(**{f: d.get(f) for f in raw})
  raise ValueError(f"Training input must contain either tokenized fields ({tok}) or raw string fields ({raw}). "
                   f"Received: {d.keys()}.")


def process_dpo_record(record: Dict[str, Any], tokenizer, max_prompt_length: int, max_response_length: int, *,
                       image_processor: Any = None) -> TrainingInput:
  """Tokenises one record (or a batch of records) with keys prompts / chosen_responses / rejected_responses."""
  prompts, ch, rj = record["prompts"], record["chosen_responses"], record["rejected_responses"]
  unbatched = isinstance(prompts, (str, dict))
  if unbatched:
    prompts = [prompts]
  ch = [ch] if isinstance(ch, str) else ch
  rj = [rj] if isinstance(rj, str) else rj
  p, pm = _generate_ids_and_masks(list(prompts), tokenizer, max_prompt_length, True)
  c, cm = _generate_ids_and_masks(list(ch), tokenizer, max_response_length, False)
  r, rm = _generate_ids_and_masks(list(rj), tokenizer, max_response_length, False)
  images = record.get("images")
  if images is not None and image_processor is not None:
    images = torch.as_tensor(np.asarray(image_processor(images)))
  if unbatched:
    p, pm, c, cm, r, rm = (t.squeeze(0) for t in (p, pm, c, cm, r, rm))
  return TrainingInput(p, pm, c, cm, r, rm, images)


class DPOTrainer(peft_trainer.PeftTrainer):
  """Preference tuning on (prompt, chosen, rejected) triples; `algorithm="orpo"` needs no reference model."""

  def __init__(self, model: torch.nn.Module, ref_model: Optional[torch.nn.Module], optimizer,
               training_config: DPOTrainingConfig, tokenizer: Any = None, image_processor: Any = None):
    self.ref_model = ref_model
    self.dpo_config = training_config
    self.algorithm = training_config.algorithm
    super().__init__(model, optimizer, training_config)
    self.tokenizer = None if tokenizer is None else tokenizer_adapter.TokenizerAdapter(tokenizer)
    self.image_processor = image_processor
    self.with_loss_fn(dpo_loss_fn, has_aux=True)
    cfg = self.dpo_config
    if self.algorithm == "orpo":
      self.with_gen_model_input_fn(lambda x: {
          "train_example": x, "algorithm": "orpo", "lambda_orpo": cfg.lambda_orpo,
          "label_smoothing": cfg.label_smoothing, "enable_prompt_loss_orpo": cfg.enable_prompt_loss_orpo,
          "average_log_prob_orpo": cfg.average_log_prob_orpo})
    else:
      self.with_gen_model_input_fn(lambda x: {
          "train_example": x, "algorithm": "dpo", "beta": cfg.beta, "label_smoothing": cfg.label_smoothing,
          "enable_prompt_loss_orpo": False, "average_log_prob_orpo": False})
    self._has_aux = True
    self._ref_model_exists = ref_model is not None
    self._aux_metrics_to_log = {"rewards/chosen": np.mean, "rewards/rejected": np.mean, "rewards/margin": np.mean,
                                "rewards/accuracy": np.mean, "log_probs/chosen": np.mean,
                                "log_probs/rejected": np.mean}
    if self.algorithm == "orpo":
      self._aux_metrics_to_log["odds_ratio"] = np.mean

  def _prepare_inputs(self, training_input: Any) -> TrainExample:
    if isinstance(training_input, TrainExample):
      return training_input
    if isinstance(training_input, dict):
      training_input = _preprocess_dict(training_input)
    if isinstance(training_input, DataInput):
      if self.tokenizer is None:
        raise ValueError("Tokenizer must be provided if training input is not tokenized.")
      mp, mr = self.dpo_config.max_prompt_length, self.dpo_config.max_response_length
      if mp is None or mr is None:
        raise ValueError("max_prompt_length and max_response_length must be provided if training input is not "
                         f"tokenized. Received: max_prompt_length={mp}, max_response_length={mr}.")
      training_input = process_dpo_record(
          {"prompts": training_input.prompts, "images": training_input.images,
           "chosen_responses": training_input.chosen_responses,
           "rejected_responses": training_input.rejected_responses},
          self.tokenizer, mp, mr, image_processor=self.image_processor)
    ti = training_input
    dev = self._device
    t = lambda x: torch.as_tensor(np.asarray(x) if not isinstance(x, torch.Tensor) else x).to(dev)
    prompt_ids = torch.cat([t(ti.prompt_ids), t(ti.prompt_ids)], 0)
    prompt_mask = torch.cat([t(ti.prompt_mask), t(ti.prompt_mask)], 0)
    comp_ids = torch.cat([t(ti.chosen_ids), t(ti.rejected_ids)], 0)
    comp_mask = torch.cat([t(ti.chosen_mask), t(ti.rejected_mask)], 0)
    input_ids = torch.cat([prompt_ids, comp_ids], 1).long()
    mask = torch.cat([prompt_mask, comp_mask], 1)
    images = ti.images
    if images is not None:
      images = torch.cat([t(images), t(images)], 0)
    # rows without padding need no explicit mask: the plain causal path runs on the flash kernels
    attn = None if bool(mask.bool().all()) else sft_utils.make_causal_attn_mask(mask)
    positions = sft_utils.build_positions_from_mask(mask)
    keep = comp_ids.shape[1]
    rc = rr = None
    if self._ref_model_exists:
      with torch.no_grad():
        rc, rr, _ = compute_logps(self.ref_model, input_ids, positions, attn, keep, comp_mask, images)
      rc, rr = rc.detach(), rr.detach()
    return TrainExample(input_ids, positions, attn, rc, rr, comp_mask, keep, images, mask)

  def _post_process_train_step(self, aux: Any) -> None:
    buf = self._buffered_train_metrics
    assert buf is not None
    for name, op in self._aux_metrics_to_log.items():
      if name in aux and name not in buf.additional_metrics:   # LossOutput aux is buffered by the base class
        buf.additional_metrics[name] = ([aux[name]], op)

  def _post_process_eval_step(self, aux: Any) -> None:
    buf = self._buffered_eval_metrics
    assert buf is not None
    for name, op in self._aux_metrics_to_log.items():
      if name in aux and name not in buf.additional_metrics:
        buf.additional_metrics[name] = ([aux[name]], op)


DpoTrainingConfig = DPOTrainingConfig
DpoTrainer = DPOTrainer
ORPOTrainingConfig = DPOTrainingConfig
ORPOTrainer = DPOTrainer
OrpoTrainingConfig = DPOTrainingConfig
OrpoTrainer = DPOTrainer
