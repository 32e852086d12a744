"""Sampler service protocol (tunix/experimental/rollout/sampler.py:30-223): async `sample`,
pause / resume, the destination-side weight-sync phases, KV-cache migration and load info."""
from __future__ import annotations

import dataclasses
from typing import Any, List, Optional, Protocol, Sequence, runtime_checkable

import numpy as np

from ..common import datatypes


@dataclasses.dataclass(frozen=True, kw_only=True)
class SamplingParams:
  max_tokens: int = 64
  temperature: float = 1.0
  top_p: Optional[float] = None
  top_k: Optional[int] = None
  seed: Optional[int] = None
  return_logprobs: bool = False
  return_logits: bool = False
  beam_size: Optional[int] = None


@dataclasses.dataclass(kw_only=True)
class SamplingRequest(datatypes.Request):
  prompt: Any
  sampling_params: Optional[SamplingParams] = None


@dataclasses.dataclass(kw_only=True)
class SamplingResponse(datatypes.Response):
  text: str = ""
  prompt_token_ids: np.ndarray = dataclasses.field(default_factory=lambda: np.zeros(0, np.int32))
  token_ids: np.ndarray = dataclasses.field(default_factory=lambda: np.zeros(0, np.int32))
  logprobs: Optional[np.ndarray] = None
  finish_reason: str = "stop"          # stop | length | cancelled | error
  routed_experts: Any = None

  def __post_init__(self):
    if self.logprobs is not None and self.logprobs.shape != self.token_ids.shape:
      raise ValueError(f"logprobs shape {self.logprobs.shape} != token_ids shape {self.token_ids.shape}")


WeightSyncRequest = datatypes.WeightSyncRequest


@dataclasses.dataclass(kw_only=True)
class LoadInfo(datatypes.Response):
  num_requests_waiting: int = 0
  num_requests_running: int = 0
  kv_cache_usage_perc: float = 0.0


@runtime_checkable
class Sampler(Protocol):
  def initialize(self) -> None: ...
  async def start(self, **kwargs) -> Any: ...
  async def stop(self, **kwargs) -> Any: ...
  async def pause(self, **kwargs) -> Any: ...
  async def resume(self, **kwargs) -> Any: ...
  async def get_mesh(self, **kwargs) -> Any: ...
  async def sample(self, sampling_requests: Sequence[Any], **kwargs) -> List[SamplingResponse]: ...
  async def bind_weight_sync(self, **kwargs) -> Any: ...
  async def get_weight_sync_metadata(self, **kwargs) -> Any: ...
  async def pre_weight_sync(self, sync_request: Any = None, **kwargs) -> Any: ...
  async def weight_sync(self, sync_request: Any = None, **kwargs) -> Any: ...
  async def post_weight_sync(self, sync_request: Any = None, **kwargs) -> Any: ...
  async def abort_weight_sync(self, sync_request: Any = None, **kwargs) -> Any: ...
  async def get_weight_sync_status(self, **kwargs) -> Any: ...
  async def migrate_kv_cache(self, target: Any = None, **kwargs) -> Any: ...
  async def get_load_info(self, **kwargs) -> LoadInfo: ...
