"""One rollout request -> one `RolloutResponse` on the worker side
(tunix/experimental/rollout/collector.py:30-200): runs the multi-turn episode through the
agentic `TrajectoryCollectEngine` with the sampler service as the model, or, without an
environment, a single sampling call."""
from __future__ import annotations

import asyncio
from types import SimpleNamespace
from typing import Any, Optional

import numpy as np

from ...rl.agentic.agents import model_agent
from ...rl.agentic.trajectory import trajectory_collect_engine
from ..common import datatypes
from . import sampler as sampler_lib


class TrajectoryCollectorEngine:
  def __init__(self, traj_id: str, request: datatypes.RolloutRequest, sampler: sampler_lib.Sampler,
               env_client: Any = None, agent: Any = None, tokenizer: Any = None, chat_parser: Any = None):
    self.traj_id, self.request, self.sampler = traj_id, request, sampler
    self.env, self.agent, self.tokenizer, self.chat_parser = env_client, agent, tokenizer, chat_parser
    self._cancelled = False

  def cancel(self) -> None:
    self._cancelled = True

  def _params(self, max_tokens: Optional[int] = None) -> sampler_lib.SamplingParams:
    kw = dict(self.request.generation_kwargs)
    return sampler_lib.SamplingParams(
        max_tokens=int(max_tokens or kw.get("max_generation_steps") or kw.get("max_tokens") or 64),
        temperature=float(kw.get("temperature", 1.0)), top_p=kw.get("top_p"), top_k=kw.get("top_k"),
        seed=kw.get("seed"), return_logprobs=True)

  async def _model_call(self, messages, env=None, max_generation_steps=None, **kw):
    prompt = self.chat_parser.parse(messages=messages, add_generation_prompt=True, is_first_msg=True) \
        if self.chat_parser is not None else messages
    rs = await self.sampler.sample([sampler_lib.SamplingRequest(request_id=self.request.request_id, prompt=prompt,
                                                                sampling_params=self._params(max_generation_steps))])
    r = rs[0]
    if r.error is not None:
      raise RuntimeError(f"sampling failed: {r.error.error_type}: {r.error.message}")
    self._version = r.metadata.get("policy_version", self.request.target_policy_version)
    return SimpleNamespace(text=[r.text], tokens=[r.token_ids], logprobs=[r.logprobs] if r.logprobs is not None else None,
                           left_padded_prompt_tokens=np.asarray(r.prompt_token_ids)[None])

  async def run(self) -> datatypes.RolloutResponse:
    req = self.request
    self._version = req.target_policy_version
    try:
      if self.env is None:                       # plain completion
        out = await self._model_call(req.prompt if not isinstance(req.prompt, str) or self.chat_parser is None
                                     else [{"role": "user", "content": req.prompt}])
        toks = np.asarray(out.tokens[0], np.int32)
        seg = datatypes.TokenSegment(source="assistant", tokens=toks, loss_mask=np.ones(len(toks), np.int32),
                                     logps=np.asarray(out.logprobs[0], np.float32) if out.logprobs else None)
        return datatypes.RolloutResponse(request_id=req.request_id, prompt_id=req.prompt_id, status="SUCCEEDED",
                                         prompt_tokens=np.asarray(out.left_padded_prompt_tokens[0], np.int32),
                                         segments=[seg], policy_version=self._version, metadata=dict(req.metadata))
      agent = self.agent or model_agent.ModelAgent("")
      if hasattr(self.env, "max_steps"):
        self.env.max_steps = min(self.env.max_steps, req.max_turns) if self.env.max_steps else req.max_turns
      eng = trajectory_collect_engine.TrajectoryCollectEngine(
          agent, self.env, model_call=self._model_call, tokenizer=self.tokenizer, chat_parser=self.chat_parser,
          max_response_length=req.generation_kwargs.get("max_response_length"))
      traj = await eng.collect("Trajectory")
      resp = datatypes.RolloutResponse.from_trajectory(traj, request_id=req.request_id, prompt_id=req.prompt_id,
                                                       policy_version=self._version)
      resp.metadata.update(req.metadata)
      return resp
    except asyncio.CancelledError:
      return datatypes.RolloutResponse(request_id=req.request_id, prompt_id=req.prompt_id, status="CANCELLED",
                                       metadata=dict(req.metadata),
                                       error=datatypes.ErrorInfo(error_type="Cancelled", message="rollout cancelled",
                                                                 retryable=True))
    except Exception as e:
      return datatypes.RolloutResponse(request_id=req.request_id, prompt_id=req.prompt_id, status="FAILED",
                                       metadata=dict(req.metadata), error=datatypes.ErrorInfo.from_exception(e))
