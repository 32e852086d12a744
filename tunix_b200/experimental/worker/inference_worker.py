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


def _as_array(x: Any) -> np.ndarray:
  return x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)


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

  def _pair(self, req: Any):
    """(prompt ids [B, P], completion ids [B, C]) of a request DTO or of anything with prompt_ids / completion_ids.
    Rows must already be padded to one width: a ragged list is a caller error, not something to re-pad here."""
    if isinstance(req, (datatypes.LogprobsRequest, datatypes.ScoreRequest)):
      p, c = req.prompt_tokens, req.completion_tokens
    else:
      p, c = req.prompt_ids, req.completion_ids
    ragged = "prompt and completion ids must be padded [batch, length] arrays with the same batch size"
    try:
      p, c = _as_array(p), _as_array(c)
    except ValueError as e:                       # numpy refuses rows of different lengths
      raise ValueError(ragged) from e
    if p.dtype == object or c.dtype == object or p.ndim != 2 or c.ndim != 2 or p.shape[0] != c.shape[0]:
      raise ValueError(ragged)
    return torch.from_numpy(p.astype(np.int64)), torch.from_numpy(c.astype(np.int64))

  def _chunks(self, m: torch.nn.Module, p: torch.Tensor, c: torch.Tensor):
    dev = next(m.parameters()).device
    step = self._mb or max(1, p.shape[0])
    for i in range(0, p.shape[0], step):
      yield p[i:i + step].to(dev), c[i:i + step].to(dev)

  def _answer(self, fn):
    try:
      out = fn()
    except Exception as e:
      self._last_error = f"{type(e).__name__}: {e}"
      raise
    self._last_error = None
    return out

  @torch.no_grad()
  def per_token_logps(self, items: Any = None, request: Optional[datatypes.LogprobsRequest] = None, temperature: float = 1.0,
                      model_role: str = "reference", **kw) -> datatypes.LogprobsResponse:
    """`items` is a LogprobsRequest or anything with prompt_ids / completion_ids (a TrainExample)."""
    req = request or items
    rid = ""
    if isinstance(req, datatypes.LogprobsRequest):
      temperature, model_role, rid = req.temperature, req.model_role, req.request_id

    def run():
      if not temperature > 1e-5:
        raise ValueError(f"temperature must be strictly positive, got {temperature}")
      m = self._model(model_role)
      p, c = self._pair(req)
      outs = [rl_common.compute_per_token_logps(m, pc, cc, self._pad, self._eos, stop_gradient=True, temperature=temperature)
              for pc, cc in self._chunks(m, p, c)]
      lp = torch.cat([o[0] if isinstance(o, tuple) else o for o in outs], 0)
      return datatypes.LogprobsResponse(request_id=rid, per_token_logps=lp.float().cpu().numpy())
    return self._answer(run)

  compute_logps = per_token_logps

  @torch.no_grad()
  def score(self, items: Any = None, request: Optional[datatypes.ScoreRequest] = None, model_role: str = "reward",
            **kw) -> datatypes.ScoreResponse:
    """One score per row. A model with a per-token head is read at the last valid completion token (the first EOS,
    or the last non-pad token of a completion without one)."""
    req = request or items
    rid = ""
    if isinstance(req, datatypes.ScoreRequest):
      model_role, rid = req.model_role, req.request_id

    def run():
      m = self._model(model_role)
      p, c = self._pair(req)
      outs = []
      for pc, cc in self._chunks(m, p, c):
        scores = rl_common.compute_score(m, pc, cc, self._pad, self._eos, stop_gradient=True).float()
        if scores.dim() > 1:
          scores = scores[:, -cc.shape[1]:]
          valid = rl_common.make_completion_mask(cc, self._eos).bool() & ((cc != self._pad) | (cc == self._eos))
          last = valid.long().sum(-1).clamp(min=1) - 1
          scores = scores.gather(-1, last[:, None]).squeeze(-1)
        outs.append(scores)
      return datatypes.ScoreResponse(request_id=rid, scores=torch.cat(outs, 0).cpu().numpy())
    return self._answer(run)
