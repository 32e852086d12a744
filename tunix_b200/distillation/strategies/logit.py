"""Logit distillation: alpha * tau^2 * KL(teacher || student) at temperature tau plus
(1 - alpha) * cross entropy, with optional restriction to the teacher's top-k logits
(tunix/distillation/strategies/logit.py:28-169)."""
from __future__ import annotations

import torch
import torch.nn.functional as F

from .base_strategy import BaseStrategy, softmax_cross_entropy


class LogitStrategy(BaseStrategy):
  def __init__(self, student_forward_fn, teacher_forward_fn, labels_fn, temperature: float = 2.0,
               alpha: float = 0.5, distill_top_k: int = 0):
    super().__init__(student_forward_fn, teacher_forward_fn, labels_fn)
    if temperature <= 0:
      raise ValueError(f"Temperature must be a positive number, got {temperature}")
    if not 0.0 <= alpha <= 1.0:
      raise ValueError(f"Alpha must be a float between 0.0 and 1.0, got {alpha}")
    self.temperature, self.alpha, self.distill_top_k = float(temperature), alpha, int(distill_top_k)

  def compute_eval_loss(self, student_output, labels):
    return softmax_cross_entropy(student_output, labels).mean(), {}

  def compute_loss(self, student_output, teacher_output, labels):
    s, t = student_output.float(), teacher_output.float()
    sk, tk = s, t
    if self.distill_top_k > 0:
      tk, idx = torch.topk(t, self.distill_top_k, dim=-1)
      sk = s.gather(-1, idx)
    log_ps = F.log_softmax(sk / self.temperature, dim=-1)
    log_pt = F.log_softmax(tk / self.temperature, dim=-1)
    pt = log_pt.exp()
    kl = (pt * (torch.where(pt > 0, log_pt, torch.zeros_like(log_pt)) - log_ps)).sum(-1)
    soft = (kl * self.temperature ** 2).mean()
    hard = softmax_cross_entropy(s, labels).mean()
    with torch.no_grad():
      teacher = softmax_cross_entropy(t, labels).mean()
    loss = self.alpha * soft + (1.0 - self.alpha) * hard
    return loss, {"distill/soft_loss": soft.detach(), "distill/hard_loss": hard.detach(),
                  "distill/kl_div": kl.mean().detach(), "distill/teacher_loss": teacher}
