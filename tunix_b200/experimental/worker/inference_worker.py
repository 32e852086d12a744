"""Worker hosting frozen models for scoring (tunix/experimental/worker/inference_worker.py:30-250):
reference per-token log-probs, reward-model scores, critic values."""
from __future__ import annotations

from typing import Any, Dict, Optional

import numpy as np
import torch

from ...rl import common as rl_common
from ..common import datatypes
from . import abstract_worker

WorkerState = datatypes.WorkerState


class InferenceWorker(abstract_worker.Worker):
  def __init__(self, models: Dict[str, torch.nn.Module], *, pad_id: int = 0, eos_id: int = 2,
               worker_id: str = "inference_worker", micro_batch_size: Optional[int] = None):
    self._models, self._pad, self._eos = dict(models), pad_id, eos_id
    self._worker_id, self._mb = worker_id, micro_batch_size
    self._state = WorkerState.PENDING
    self._last_error: Optional[str] = None

  def initialize(self) -> datatypes.Response:
    with self._phase(WorkerState.INITIALIZING):
      for m in self._models.values():
        m.eval()
    return datatypes.Response()

  def compile(self, dummy_data: Any = None) -> datatypes.Response:
    with self._phase(WorkerState.COMPILING):
      pass
    return datatypes.Response()

  def start(self) -> datatypes.Response:
    return datatypes.Response()

  def stop(self) -> datatypes.Response:
    self._state = WorkerState.STOPPED
    return datatypes.Response()

  def info(self) -> datatypes.WorkerInfo:
    return datatypes.WorkerInfo(worker_id=self._worker_id, roles=frozenset(self._models), resources={})

  def heartbeat(self) -> datatypes.HealthReport:
    return datatypes.HealthReport(state=self.state, last_error=self._last_error)

  def _model(self, role: str) -> torch.nn.Module:
    if role not in self._models:
      raise KeyError(f"no model hosted for role {role!r}; hosted: {sorted(self._models)}")
    return self._models[role]

  @torch.no_grad()
  def per_token_logps(self, items: Any = None, request: Optional[datatypes.LogprobsRequest] = None, temperature: float = 1.0,
                      model_role: str = "reference", **kw) -> datatypes.LogprobsResponse:
    """`items` is a LogprobsRequest or anything with prompt_ids / completion_ids (a TrainExample)."""
    req = request or items
    if isinstance(req, datatypes.LogprobsRequest):
      p, c, temperature, model_role = req.prompt_tokens, req.completion_tokens, req.temperature, req.model_role
      rid = req.request_id
    else:
      p, c, rid = req.prompt_ids, req.completion_ids, ""
    m = self._model(model_role)
    dev = next(m.parameters()).device
    p, c = torch.as_tensor(np.asarray(p)).long().to(dev), torch.as_tensor(np.asarray(c)).long().to(dev)
    outs = []
    step = self._mb or p.shape[0]
    for i in range(0, p.shape[0], step):
      outs.append(rl_common.compute_per_token_logps(m, p[i:i + step], c[i:i + step], self._pad, self._eos,
                                                    stop_gradient=True, temperature=temperature))
    lp = torch.cat([o[0] if isinstance(o, tuple) else o for o in outs], 0)
    return datatypes.LogprobsResponse(request_id=rid, per_token_logps=lp.float().cpu().numpy())

  @torch.no_grad()
  def score(self, items: Any = None, request: Optional[datatypes.ScoreRequest] = None, model_role: str = "reward",
            **kw) -> datatypes.ScoreResponse:
    req = request or items
    if isinstance(req, datatypes.ScoreRequest):
      p, c, model_role, rid = req.prompt_tokens, req.completion_tokens, req.model_role, req.request_id
    else:
      p, c, rid = req.prompt_ids, req.completion_ids, ""
    m = self._model(model_role)
    dev = next(m.parameters()).device
    p, c = torch.as_tensor(np.asarray(p)).long().to(dev), torch.as_tensor(np.asarray(c)).long().to(dev)
    scores = rl_common.compute_score(m, p, c, self._pad, self._eos, stop_gradient=True)
    scores = scores.float()
    if scores.dim() > 1:                      # per-token scores: take the last completion token
      last = (c != self._pad).long().sum(-1).clamp(min=1) - 1
      scores = scores.gather(-1, last[:, None]).squeeze(-1)
    return datatypes.ScoreResponse(request_id=rid, scores=scores.cpu().numpy())
