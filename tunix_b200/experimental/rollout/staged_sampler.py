"""What every in-process `Sampler` service shares: admission control, load counters and the destination side
of a weight-sync round. Engine adapters (`native_sampler_adapter`, `vanilla_sampler_adapter`,
`inprocess_vllm_sampler_adapter`) derive from `StagedSampler` and supply three things: how to generate for a
batch of requests that share sampling parameters, which tensors are being served, and how a staged copy of them
is published into the engine.

Weight sync follows the destination contract of the coordinator
(tunix/experimental/rollout/vanilla_sampler_adapter.py:40-342 plays this role in the reference):

  bind    a STAGING copy of the serving parameters is attached to the transport, which will write into it;
  pre     admission closes and running generations drain - they finish on the old weights;
  sync    bookkeeping only (the transport has filled staging);
  post    staging is published into the engine in one pass under the generation lock, the policy version is
          bumped, admission reopens;
  abort   admission reopens on the old parameters.

Phases are serialised by one lock and deduplicated by the round tracker, so an abort that overtakes a timed-out
phase cannot interleave with it and a retried phase runs once. Requests that arrive while admission is closed are
answered `cancelled` with a retryable error rather than queued, so the router can send them elsewhere.
"""
from __future__ import annotations

import abc
import asyncio
import collections
import threading
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch

from ...generate import tokenizer_adapter as tok_adapter
from ..common import datatypes
from ..orchestrator import peer_memory_handler, weight_sync, weight_sync_coordinator as wsc
from . import sampler as sampler_lib

_DRAIN_POLL_S = 0.005


class StagedSampler(abc.ABC):

  def __init__(self, tokenizer: Any, *, handler: Optional[weight_sync.WeightSyncHandler] = None,
               worker_id: str = "sampler0", rank: int = 0, eos_ids: Optional[Sequence[int]] = None):
    self._tok = tokenizer if isinstance(tokenizer, tok_adapter.TokenizerAdapter) else \
        tok_adapter.TokenizerAdapter(tokenizer)
    self._handler, self._worker_id, self._rank = handler, worker_id, rank
    self._eos = list(eos_ids) if eos_ids else [self._tok.eos_id()]
    self._gen_lock = threading.Lock()          # generation vs. publish
    self._phase_lock = asyncio.Lock()
    self._admitting = True
    self._running = 0
    self._waiting = 0
    self._staging: Optional[Dict[str, torch.Tensor]] = None
    self._tracker = wsc.WorkerRoundTracker()
    self.policy_version = 0

  # ---- what an engine adapter supplies -------------------------------------------------------
  @abc.abstractmethod
  def initialize(self) -> None:
    """Builds the engine (idempotent)."""

  @abc.abstractmethod
  def _generate_batch(self, reqs: Sequence[sampler_lib.SamplingRequest], params: sampler_lib.SamplingParams
                      ) -> List[sampler_lib.SamplingResponse]:
    """Blocking generation for requests that share `params`. Called on a worker thread under the generation lock."""

  @abc.abstractmethod
  def _serving(self) -> Dict[str, torch.Tensor]:
    """The tensors a weight sync replaces, by name."""

  def _publish(self, staging: Dict[str, torch.Tensor]) -> None:
    """Staging -> serving. Default: in-place copies (engines that read the same tensors see them at once)."""
    with torch.no_grad():
      for name, dst in self._serving().items():
        dst.copy_(staging[name])

  def _cache_usage_percent(self) -> float:
    return 0.0

  # ---- lifecycle -------------------------------------------------------------------------------
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
    return sampler_lib.LoadInfo(num_requests_waiting=self._waiting, num_requests_running=self._running,
                                kv_cache_usage_perc=self._cache_usage_percent())

  async def migrate_kv_cache(self, target: Any = None, **kwargs):
    """Sequences are re-prefilled on the target instead of shipping pages: prompts are short relative to
    generations and the prefix is shared per group."""
    return {"migrated": 0, "strategy": "recompute"}

  # ---- sampling ----------------------------------------------------------------------------------
  def prompt_ids(self, prompt: Any) -> List[int]:
    """Token ids of a prompt given as text (one BOS in front) or as ids."""
    if not isinstance(prompt, str):
      return [int(t) for t in np.asarray(prompt).reshape(-1)]
    ids = list(self._tok.encode(prompt))
    bos = self._tok.bos_id()
    return list(self._tok.dedup_bos_ids([bos] + ids)) if bos else ids

  def response(self, req: sampler_lib.SamplingRequest, prompt: Sequence[int], tokens: np.ndarray,
               logprobs: Optional[np.ndarray], hit_eos: bool, version: int) -> sampler_lib.SamplingResponse:
    tokens = np.asarray(tokens, np.int32)
    return sampler_lib.SamplingResponse(
        request_id=req.request_id, text=self._tok.decode([t for t in tokens.tolist() if t not in self._eos]),
        prompt_token_ids=np.asarray(prompt, np.int32), token_ids=tokens, logprobs=logprobs,
        finish_reason="stop" if hit_eos else "length", metadata={**req.metadata, "policy_version": version})

  def _generate(self, reqs: Sequence[sampler_lib.SamplingRequest]) -> List[sampler_lib.SamplingResponse]:
    """Requests are bucketed by their sampling parameters (engines take one setting per batch); the answers
    come back in request order."""
    self.initialize()
    buckets: Dict[sampler_lib.SamplingParams, List[int]] = collections.OrderedDict()
    for i, r in enumerate(reqs):
      buckets.setdefault(r.sampling_params or sampler_lib.SamplingParams(), []).append(i)
    answers: List[Optional[sampler_lib.SamplingResponse]] = [None] * len(reqs)
    with self._gen_lock:
      for params, members in buckets.items():
        for i, ans in zip(members, self._generate_batch([reqs[i] for i in members], params)):
          answers[i] = ans
    return answers      # type: ignore[return-value]

  def _refused(self, reqs, why: str, error_type: str, reason: str, retryable: bool):
    err = datatypes.ErrorInfo(error_type=error_type, retryable=retryable, message=why)
    return [sampler_lib.SamplingResponse(request_id=r.request_id, finish_reason=reason, error=err) for r in reqs]

  async def sample(self, sampling_requests, **kwargs) -> List[sampler_lib.SamplingResponse]:
    reqs = [r if isinstance(r, sampler_lib.SamplingRequest) else sampler_lib.SamplingRequest(prompt=r)
            for r in sampling_requests]
    if not reqs:
      return []
    if not self._admitting:
      return self._refused(reqs, "sampler is paused for a weight sync", "AdmissionClosed", "cancelled", True)
    self._running += len(reqs)
    try:
      return await asyncio.get_running_loop().run_in_executor(None, self._generate, reqs)
    except Exception as e:  # noqa: BLE001 - reported per request
      err = datatypes.ErrorInfo.from_exception(e)
      return [sampler_lib.SamplingResponse(request_id=r.request_id, finish_reason="error", error=err) for r in reqs]
    finally:
      self._running -= len(reqs)

  # ---- weight-sync destination ---------------------------------------------------------------
  @property
  def work_unit(self) -> weight_sync.WorkUnitId:
    return weight_sync.WorkUnitId(job_name="rollout", job_replica_id=self._worker_id, data_replica_idx=self._rank)

  async def bind_weight_sync(self, **kwargs) -> None:
    if self._staging is None:
      self._staging = {n: torch.empty_like(p) for n, p in self._serving().items()}
    if self._handler is not None and hasattr(self._handler, "attach"):
      self._handler.attach(self.work_unit, self._staging)

  async def get_weight_sync_metadata(self, **kwargs):
    return [peer_memory_handler.manifest_of(self.work_unit, self._staging or self._serving())]

  async def get_weight_sync_status(self, **kwargs):
    return self._tracker.report()

  async def _phase(self, sync_request: Any, name: str, work) -> None:
    async with self._phase_lock:
      if self._tracker.admit(sync_request, name):
        await work()
        self._tracker.complete(sync_request, name)

  async def pre_weight_sync(self, sync_request: Any = None, **kwargs):
    async def drain():
      self._admitting = False
      while self._running > 0:
        await asyncio.sleep(_DRAIN_POLL_S)
    await self._phase(sync_request, "prepared", drain)

  async def weight_sync(self, sync_request: Any = None, **kwargs):
    async def nothing():
      return None
    await self._phase(sync_request, "h2d_done", nothing)

  async def post_weight_sync(self, sync_request: Any = None, **kwargs):
    async def publish():
      with self._gen_lock:
        self._publish(self._staging)
        self.policy_version = int(getattr(sync_request, "policy_version", self.policy_version + 1))
      self._admitting = True
    await self._phase(sync_request, "committed", publish)

  async def abort_weight_sync(self, sync_request: Any = None, **kwargs):
    async def reopen():
      self._admitting = True
    await self._phase(sync_request, "aborted", reopen)


def lora_aware_parameters(model: torch.nn.Module) -> Dict[str, torch.Tensor]:
  """All parameters, or only the adapter parameters when the model carries LoRA adapters (the base stays put)."""
  has_lora = any(getattr(p, "is_lora", False) for p in model.parameters())
  return {n: p for n, p in model.named_parameters() if getattr(p, "is_lora", False) or not has_lora}
