"""Hosts the frozen models of an RL cluster - reference policy, critic, reward model - and answers
log-probability / value / reward queries (tunix/rl/inference/inference_worker.py:22-100)."""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch

from .. import common


class InferenceWorker:

  def __init__(self, models: Dict[str, torch.nn.Module]):
    for k in models:
      if k not in ("critic", "reference", "reward"):
        raise ValueError(f"Model role {k} is not supported. Supported models are critic, reference and reward.")
    self._models = dict(models)

  def get_rewards(self, prompt_tokens, completion_tokens, pad_id: int, eos_id: int):
    m = self._models.get("reward")
    if m is None:
      raise ValueError("Reward model is not available.")
    return common.compute_score(m, prompt_tokens, completion_tokens, pad_id, eos_id)

  def get_ref_per_token_logps(self, prompt_tokens, completion_tokens, pad_id: int, eos_id: int,
                              completion_mask=None, segment_ids=None, segment_positions=None, temperature: float = 1.0,
                              chunk_size: int = 0):
    m = self._models.get("reference")
    if m is None:
      raise ValueError("Reference model is not available.")
    return common.compute_per_token_logps(m, prompt_tokens, completion_tokens, pad_id, eos_id, stop_gradient=True,
                                          segment_ids=segment_ids, segment_positions=segment_positions,
                                          temperature=temperature, chunk_size=chunk_size)

  def get_values(self, prompt_tokens, completion_tokens, pad_id: int, eos_id: int, completion_mask=None):
    m = self._models.get("critic")
    if m is None:
      raise ValueError("Critic model is not available.")
    return common.compute_score(m, prompt_tokens, completion_tokens, pad_id, eos_id)

  def get_model(self, role: str) -> torch.nn.Module:
    if role not in self._models:
      raise ValueError(f"Model role {role} is not available.")
    return self._models[role]

  def update_model(self, role: str, model: torch.nn.Module) -> None:
    self._models[role] = model
