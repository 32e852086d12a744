"""`Sampler` service over the paged engine (the role of the reference's vanilla / in-process vLLM
adapters: tunix/experimental/rollout/vanilla_sampler_adapter.py:40-342).

Weight sync follows the destination contract: `bind` attaches a STAGING copy of the parameters
to the transport, `pre` pauses admission and waits for running generations, `weight_sync` is a
no-op beyond bookkeeping (the transport has written into staging), `post` publishes staging
into the serving parameters in one pass under the generation lock and resumes, `abort` resumes
on the old parameters. Phases are serialised by one lock, so an abort that overtakes a
timed-out phase cannot interleave with it."""
from __future__ import annotations

import asyncio
import threading
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ...generate import tokenizer_adapter as tok_adapter
from ...rollout import EngineConfig, PagedEngine
from ..common import datatypes
from ..orchestrator import peer_memory_handler, weight_sync, weight_sync_coordinator as wsc
from . import sampler as sampler_lib


class NativeSamplerAdapter:
  def __init__(self, model: torch.nn.Module, tokenizer: Any, *, engine_config: Optional[EngineConfig] = None,
               handler: Optional[weight_sync.WeightSyncHandler] = None, worker_id: str = "sampler0", rank: int = 0,
               eos_ids: Optional[Sequence[int]] = None):
    self._model = model
    self._tok = tokenizer if isinstance(tokenizer, tok_adapter.TokenizerAdapter) else \
        tok_adapter.TokenizerAdapter(tokenizer)
    self._cfg = engine_config or EngineConfig()
    self._handler, self._worker_id, self._rank = handler, worker_id, rank
    self._eos = list(eos_ids) if eos_ids else [self._tok.eos_id()]
    self._engine: Optional[PagedEngine] = None
    self._gen_lock = threading.Lock()          # generation vs. publish
    self._phase_lock = asyncio.Lock()
    self._admitting = True
    self._running = 0
    self._waiting = 0
    self._staging: Optional[Dict[str, torch.Tensor]] = None
    self._tracker = wsc.WorkerRoundTracker()
    self.policy_version = 0

  # ---- lifecycle -----------------------------------------------------------------------------
  def initialize(self) -> None:
    if self._engine is None:
      self._engine = PagedEngine(self._model, self._cfg)

  async def start(self, **kwargs):
    self.initialize()
    self._admitting = True

  async def stop(self, **kwargs):
    self._admitting = False

  async def pause(self, **kwargs):
    self._admitting = False

  async def resume(self, **kwargs):
    self._admitting = True

  async def get_mesh(self, **kwargs):
    return None

  async def get_load_info(self, **kwargs) -> sampler_lib.LoadInfo:
    used = 0.0
    if self._engine is not None:
      a = self._engine.cache.allocator
      used = 100.0 * (1.0 - a.free_pages / max(a.num_pages, 1))
    return sampler_lib.LoadInfo(num_requests_waiting=self._waiting, num_requests_running=self._running,
                                kv_cache_usage_perc=used)

  async def migrate_kv_cache(self, target: Any = None, **kwargs):
    """Sequences are re-prefilled on the target instead of shipping pages: prompts are short
    relative to generations and the prefix is shared per group."""
    return {"migrated": 0, "strategy": "recompute"}

  # ---- sampling ------------------------------------------------------------------------------
  def _ids(self, prompt: Any) -> List[int]:
    if isinstance(prompt, str):
      ids = list(self._tok.encode(prompt))
      bos = self._tok.bos_id()
      return list(self._tok.dedup_bos_ids([bos] + ids)) if bos else ids
    return [int(t) for t in np.asarray(prompt).reshape(-1)]

  def _generate(self, reqs: Sequence[sampler_lib.SamplingRequest]) -> List[sampler_lib.SamplingResponse]:
    self.initialize()
    p0 = reqs[0].sampling_params or sampler_lib.SamplingParams()
    ids = [self._ids(r.prompt) for r in reqs]
    with self._gen_lock:
      version = self.policy_version
      res = self._engine.generate(ids, p0.max_tokens, temperature=p0.temperature, greedy=p0.temperature == 0.0,
                                  seed=p0.seed or 0, eos_ids=self._eos)
    out = []
    for r, p, t, lp, why in zip(reqs, ids, res.tokens, res.logprobs, res.finish_reasons):
      out.append(sampler_lib.SamplingResponse(
          request_id=r.request_id, text=self._tok.decode([x for x in t.tolist() if x not in self._eos]),
          prompt_token_ids=np.asarray(p, np.int32), token_ids=t.astype(np.int32),
          logprobs=lp if p0.return_logprobs else None, finish_reason="stop" if why == "eos" else "length",
          metadata={**r.metadata, "policy_version": version}))
    return out

  async def sample(self, sampling_requests, **kwargs) -> List[sampler_lib.SamplingResponse]:
    reqs = [r if isinstance(r, sampler_lib.SamplingRequest) else sampler_lib.SamplingRequest(prompt=r)
            for r in sampling_requests]
    if not reqs:
      return []
    if not self._admitting:
      return [sampler_lib.SamplingResponse(request_id=r.request_id, finish_reason="cancelled",
                                           error=datatypes.ErrorInfo(error_type="AdmissionClosed", retryable=True,
                                                                     message="sampler is paused for a weight sync"))
              for r in reqs]
    self._waiting += len(reqs)
    try:
      self._running += len(reqs)
      self._waiting -= len(reqs)
      return await asyncio.get_running_loop().run_in_executor(None, self._generate, reqs)
    except Exception as e:
      err = datatypes.ErrorInfo.from_exception(e)
      return [sampler_lib.SamplingResponse(request_id=r.request_id, finish_reason="error", error=err) for r in reqs]
    finally:
      self._running -= len(reqs)

  # ---- weight-sync destination ---------------------------------------------------------------
  @property
  def work_unit(self) -> weight_sync.WorkUnitId:
    return weight_sync.WorkUnitId(job_name="rollout", job_replica_id=self._worker_id, data_replica_idx=self._rank)

  def _serving(self) -> Dict[str, torch.Tensor]:
    lora = any(getattr(p, "is_lora", False) for p in self._model.parameters())
    return {n: p for n, p in self._model.named_parameters() if getattr(p, "is_lora", False) or not lora}

  async def bind_weight_sync(self, **kwargs) -> None:
    if self._staging is None:
      self._staging = {n: torch.empty_like(p) for n, p in self._serving().items()}
    if self._handler is not None and hasattr(self._handler, "attach"):
      self._handler.attach(self.work_unit, self._staging)

  async def get_weight_sync_metadata(self, **kwargs):
    return [peer_memory_handler.manifest_of(self.work_unit, self._staging or self._serving())]

  async def get_weight_sync_status(self, **kwargs):
    return self._tracker.report()

  async def pre_weight_sync(self, sync_request: Any = None, **kwargs):
    async with self._phase_lock:
      if self._tracker.admit(sync_request, "prepared"):
        self._admitting = False
        while self._running > 0:                   # drain: running generations finish on the old weights
          await asyncio.sleep(0.005)
        self._tracker.complete(sync_request, "prepared")

  async def weight_sync(self, sync_request: Any = None, **kwargs):
    async with self._phase_lock:
      if self._tracker.admit(sync_request, "h2d_done"):
        self._tracker.complete(sync_request, "h2d_done")     # the transport wrote into staging

  async def post_weight_sync(self, sync_request: Any = None, **kwargs):
    async with self._phase_lock:
      if self._tracker.admit(sync_request, "committed"):
        with self._gen_lock, torch.no_grad():
          for n, p in self._serving().items():
            p.copy_(self._staging[n])
          self.policy_version = int(getattr(sync_request, "policy_version", self.policy_version + 1))
        self._admitting = True
        self._tracker.complete(sync_request, "committed")

  async def abort_weight_sync(self, sync_request: Any = None, **kwargs):
    async with self._phase_lock:
      if self._tracker.admit(sync_request, "aborted"):
        self._admitting = True
        self._tracker.complete(sync_request, "aborted")
