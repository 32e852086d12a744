"""The in-process `Sampler` services: dense-cache ("vanilla") and in-process vLLM (over a fake engine), including
bucketing by sampling parameters, admission control and one weight-sync round."""
import asyncio
import types

import numpy as np
import torch

from tests.test_rl_grpo import ToyTokenizer, toy_model
from tunix_b200.experimental.common import datatypes
from tunix_b200.experimental.rollout import (inprocess_vllm_sampler_adapter as vllm_ad, sampler as sampler_lib,
                                             vanilla_sampler_adapter as vanilla_ad)


def _req(prompt, **params):
  return sampler_lib.SamplingRequest(prompt=prompt, sampling_params=sampler_lib.SamplingParams(**params))


def _sync_round(adapter, new_state, version):
  async def go():
    req = datatypes.WeightSyncRequest(request_id=f"s{version}", policy_version=version)
    await adapter.bind_weight_sync()
    await adapter.pre_weight_sync(req)
    assert (await adapter.sample(["a b"]))[0].finish_reason == "cancelled"      # admission is closed meanwhile
    with torch.no_grad():
      for n, t in adapter._staging.items():
        t.copy_(new_state[n])                                                    # what a transport would do
    await adapter.weight_sync(req)
    await adapter.post_weight_sync(req)
  asyncio.run(go())


def test_vanilla_adapter_generates_buckets_and_takes_new_weights():
  torch.manual_seed(0)
  model, donor = toy_model(0), toy_model(1)
  ad = vanilla_ad.VanillaSamplerAdapter(model, ToyTokenizer(), worker_id="v0")
  reqs = [_req("alpha beta", max_tokens=4, temperature=0.0, return_logprobs=True),
          _req(np.array([1, 5, 6]), max_tokens=2, temperature=0.0),
          _req("gamma", max_tokens=4, temperature=0.0, return_logprobs=True)]
  out = asyncio.run(ad.sample(reqs))
  assert [o.request_id for o in out] == [r.request_id for r in reqs]
  assert out[1].prompt_token_ids.tolist() == [1, 5, 6] and len(out[1].token_ids) <= 2 and out[1].logprobs is None
  assert out[0].logprobs is not None and out[0].logprobs.shape == out[0].token_ids.shape
  assert all(o.metadata["policy_version"] == 0 for o in out)
  greedy_before = out[0].token_ids.tolist()
  _sync_round(ad, dict(donor.named_parameters()), version=3)
  for (n, p), (_, q) in zip(model.named_parameters(), donor.named_parameters()):
    assert torch.equal(p, q), n
  again = asyncio.run(ad.sample(reqs[:1]))[0]
  assert again.metadata["policy_version"] == 3 and ad.policy_version == 3
  # the same greedy request on the donor's weights directly gives the same tokens
  direct = asyncio.run(vanilla_ad.VanillaSamplerAdapter(donor, ToyTokenizer()).sample(reqs[:1]))[0]
  assert again.token_ids.tolist() == direct.token_ids.tolist()
  assert isinstance(greedy_before, list)


class _FakeVllm:
  def __init__(self):
    self.batches, self.loaded, self.resets = [], None, 0

  def generate(self, prompts, params, use_tqdm=False):
    self.batches.append((len(prompts), params["max_tokens"] if isinstance(params, dict) else params.max_tokens))
    outs = []
    for p in prompts:
      last = p["prompt_token_ids"][-1]
      toks = [last + 1, last + 2, 2]
      lps = [{t: types.SimpleNamespace(logprob=-0.25 * (k + 1))} for k, t in enumerate(toks)]
      outs.append(types.SimpleNamespace(outputs=[types.SimpleNamespace(token_ids=toks, logprobs=lps, finish_reason="stop")]))
    return outs

  def load_weights(self, weights):
    self.loaded = dict(weights)

  def reset_prefix_cache(self):
    self.resets += 1


def test_inprocess_vllm_adapter_forwards_and_streams_weights_under_checkpoint_names():
  model, donor = toy_model(0), toy_model(1)
  llm = _FakeVllm()
  ad = vllm_ad.InprocessVllmSamplerAdapter(model, ToyTokenizer(), llm=llm, eos_ids=[2])
  reqs = [_req([1, 7], max_tokens=8, return_logprobs=True), _req([1, 9], max_tokens=4), _req([1, 3], max_tokens=8,
                                                                                          return_logprobs=True)]
  out = asyncio.run(ad.sample(reqs))
  assert sorted(llm.batches) == [(1, 4), (2, 8)]                      # one engine call per sampling setting
  assert out[0].token_ids.tolist() == [8, 9, 2] and out[0].finish_reason == "stop" and out[0].text is not None
  np.testing.assert_allclose(out[0].logprobs, [-0.25, -0.5, -0.75])
  assert out[1].logprobs is None and out[2].token_ids.tolist() == [4, 5, 2]
  _sync_round(ad, dict(donor.named_parameters()), version=1)
  assert "model.layers.0.self_attn.q_proj.weight" in llm.loaded      # exporter names, fused projections split
  assert torch.equal(model.lm_head.w if hasattr(model.lm_head, "w") else next(model.parameters()),
                     donor.lm_head.w if hasattr(donor.lm_head, "w") else next(donor.parameters()))
  assert ad.policy_version == 1
