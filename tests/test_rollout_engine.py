"""Paged continuous-batching engine on CPU: token-for-token agreement with the contiguous-cache
sampler, page accounting, prefix sharing, admission under a small cache."""
import numpy as np
import pytest
import torch

from tunix_b200.common.configs import CacheConfig
from tunix_b200.generate import sampler as sampler_lib
from tunix_b200.models.transformer import ModelConfig, Transformer
from tunix_b200.rollout import EngineConfig, PagedEngine, PageAllocator
from tunix_b200.rollout.paged_cache import OutOfPages


class IdTok:
  def encode(self, s, **k): return [int(x) for x in s.split()]
  def decode(self, ids, **k): return " ".join(str(int(i)) for i in ids)
  def bos_id(self): return None
  def eos_id(self): return 2
  def pad_id(self): return 0


def model(**kw):
  cfg = ModelConfig(num_layers=2, vocab_size=50, embed_dim=32, hidden_dim=64, num_heads=4, head_dim=8, num_kv_heads=2,
                    **kw)
  return Transformer(cfg).init_weights(seed=0, scale=0.3).eval()


def test_page_allocator():
  a = PageAllocator(4)
  p = a.alloc(3)
  q = a.share(p[:2])
  a.free(p)
  assert a.free_pages == 2 and a.refcount(p[0]) == 1
  a.free(q)
  assert a.free_pages == 4
  with pytest.raises(OutOfPages):
    a.alloc(5)
  with pytest.raises(AssertionError):
    a.free([p[0]])


@pytest.mark.parametrize("qk_norm", [False, True])
def test_greedy_matches_contiguous_sampler(qk_norm):
  m = model(use_qk_norm=qk_norm)
  prompts = [[5, 6, 7], [9, 10, 11, 12, 13, 14, 15], [20], [5, 6, 7]]
  eng = PagedEngine(m, EngineConfig(page_size=4, max_batch=8, max_seq_len=32))
  res = eng.generate(prompts, 10, greedy=True, eos_ids=[2])
  s = sampler_lib.Sampler(m, IdTok(), CacheConfig(cache_size=64, num_layers=2, num_kv_heads=2, head_dim=8))
  for p, got, lp in zip(prompts, res.tokens, res.logprobs):
    ref = s([" ".join(map(str, p))], max_generation_steps=10, eos_tokens=[2], return_logprobs=True)
    want = np.asarray(ref.tokens[0])
    # the sampler strips the EOS; the engine keeps it
    got_cmp = got[:-1] if len(got) and got[-1] == 2 else got
    assert got_cmp.tolist() == want.tolist()
    np.testing.assert_allclose(lp[:len(want)], np.asarray(ref.logprobs[0]), rtol=1e-4, atol=1e-4)
  assert eng.cache.allocator.free_pages == eng.cache.num_pages


def test_prefix_sharing_and_small_cache_admission():
  m = model()
  prompt = list(range(3, 13))               # 10 tokens: 2 full pages of 4 + a tail of 2
  # every sequence needs ceil((10 + 6) / 4) = 4 pages; 7 pages hold one group member plus one follower (4 + 2)
  eng = PagedEngine(m, EngineConfig(page_size=4, num_pages=7, max_batch=8, max_seq_len=16))
  res = eng.generate([prompt] * 5, 6, temperature=1.0, seed=4)
  assert len(res.tokens) == 5 and all(len(t) == 6 for t in res.tokens)
  assert eng.cache.allocator.free_pages == 7
  # same seed -> same draws; samples of one prompt differ from each other
  res2 = eng.generate([prompt] * 5, 6, temperature=1.0, seed=4)
  assert all(a.tolist() == b.tolist() for a, b in zip(res.tokens, res2.tokens))
  assert len({tuple(t.tolist()) for t in res.tokens}) > 1
  # shared prefix gives the same distribution as unshared: greedy outputs agree
  g1 = eng.generate([prompt] * 3, 6, greedy=True).tokens
  eng2 = PagedEngine(m, EngineConfig(page_size=4, max_batch=8, max_seq_len=16, share_prefix=False))
  g2 = eng2.generate([prompt] * 3, 6, greedy=True).tokens
  assert all(a.tolist() == b.tolist() for a, b in zip(g1, g2)) and g1[0].tolist() == g1[2].tolist()
  with pytest.raises(OutOfPages):
    PagedEngine(m, EngineConfig(page_size=4, num_pages=3, max_seq_len=16)).generate([prompt], 6)
  with pytest.raises(ValueError):
    eng.generate([prompt], 7)


def test_logprobs_match_training_forward():
  m = model()
  prompt = [4, 8, 15, 16, 23]
  eng = PagedEngine(m, EngineConfig(page_size=4, max_batch=4, max_seq_len=32))
  res = eng.generate([prompt], 7, temperature=0.8, seed=1)
  seq = torch.tensor([prompt + res.tokens[0].tolist()])
  with torch.no_grad():
    logits, _ = m(seq, None, None, None)
  lp = torch.log_softmax(logits[0, len(prompt) - 1:-1] / 0.8, -1).gather(-1, seq[0, len(prompt):, None])[:, 0]
  np.testing.assert_allclose(res.logprobs[0], lp.numpy(), rtol=1e-4, atol=1e-4)


def test_native_rollout_in_grpo_cluster():
  from tests.test_rl_grpo import ToyTokenizer, prompts_ds, reward_len, toy_model
  from tunix_b200 import optim
  from tunix_b200.common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
  from tunix_b200.common.datatypes import Role
  from tunix_b200.rl import rl_cluster
  from tunix_b200.rl.grpo import grpo_learner
  tc = RLTrainingConfig(actor_optimizer=optim.adamw(1e-2), eval_every_n_steps=100, max_steps=2, pbar_description=None)
  rc = RolloutConfig(max_tokens_to_generate=8, max_prompt_length=8, kv_cache_size=32, temperature=1.0, top_p=1.0,
                     seed=3, return_logprobs=True)
  cc = ClusterConfig(role_to_mesh={Role.ACTOR: None, Role.REFERENCE: None, Role.ROLLOUT: None},
                     rollout_engine="native", training_config=tc, rollout_config=rc)
  cluster = rl_cluster.RLCluster(actor=toy_model(), reference=toy_model(), tokenizer=ToyTokenizer(), cluster_config=cc)
  out = cluster.generate(["alpha beta gamma", "delta"])
  assert out.left_padded_prompt_tokens.shape == (2, 8) and len(out.tokens) == 2 and len(out.logprobs[0]) == len(out.tokens[0])
  # rollout log-probs agree with the trainer's recompute on the same tokens
  learner = grpo_learner.GRPOLearner(rl_cluster=cluster, algo_config=grpo_learner.GRPOConfig(num_generations=2),
                                     reward_fns=[reward_len])
  learner.train(prompts_ds(2))
  assert cluster.global_steps == 2
  ml = cluster.actor_trainer.metrics_logger
  pre = cluster.actor_trainer.metrics_prefix
  assert all(np.isfinite(ml.get_metric_history(pre, "loss", "train")))


def test_top_k_and_top_p_in_the_paged_engine():
  """top_k=1 is greedy; top-k draws stay inside the k best tokens; log-probs are those of the full distribution."""
  from tests.test_rl_grpo import toy_model
  from tunix_b200.rollout import EngineConfig, PagedEngine
  model = toy_model(0)
  eng = PagedEngine(model, EngineConfig(page_size=4, max_batch=4, max_seq_len=32, use_cuda_graphs=False))
  prompts = [[5, 6, 7], [9, 10, 11, 12], [3, 4]]
  greedy = eng.generate(prompts, 6, greedy=True, eos_ids=[63])
  k1 = eng.generate(prompts, 6, temperature=1.0, top_k=1, seed=4, eos_ids=[63])
  assert [list(t) for t in greedy.tokens] == [list(t) for t in k1.tokens]
  out = eng.generate(prompts, 6, temperature=1.3, top_k=3, top_p=0.9, seed=5, eos_ids=[63])
  for p, toks, lps in zip(prompts, out.tokens, out.logprobs):
    ids = list(p)
    for t, lp in zip(toks, lps):
      full = torch.tensor([ids])
      logits, _ = model(full, torch.arange(len(ids))[None], None, None)
      z = logits[0, -1].float() / 1.3
      assert int(t) in torch.topk(z, 3).indices.tolist()
      np.testing.assert_allclose(float(torch.log_softmax(z, -1)[int(t)]), float(lp), atol=2e-4)
      ids.append(int(t))


def test_sglang_jax_configuration_is_translated_to_engine_geometry():
  import types
  from tunix_b200.common.configs import RolloutConfig
  from tunix_b200.rl.rollout import sglang_jax_rollout as sg
  mc = types.SimpleNamespace(num_layers=4, num_kv_heads=2, head_dim=64)
  rc = RolloutConfig(max_tokens_to_generate=64, max_prompt_length=64, kv_cache_size=96,
                     rollout_sglang_jax_page_size=128, rollout_sglang_jax_context_length=512,
                     rollout_sglang_jax_max_running_requests=48, rollout_sglang_jax_chunked_prefill_size=2048,
                     rollout_sglang_jax_precompile_bs_paddings=[8, 16, 64], rollout_sglang_jax_mem_fraction_static=0.5)
  g = sg.engine_geometry(rc, mc, device_memory_bytes=1 << 30)
  assert g["page_size"] == 64 and g["max_seq_len"] == 512 and g["max_batch"] == 48
  assert g["max_prefill_tokens"] == 2048 and g["warm_buckets"] == [8, 16, 48]
  per_page = 64 * 2 * 4 * 2 * 64 * 2
  assert g["num_pages"] == min(48 * 8, (1 << 29) // per_page)
  small = sg.engine_geometry(RolloutConfig(max_tokens_to_generate=8, max_prompt_length=8, kv_cache_size=16,
                                           rollout_sglang_jax_page_size=4, rollout_sglang_jax_chunked_prefill_size=-1), mc)
  assert small["page_size"] == 8 and small["max_seq_len"] == 16 and "max_prefill_tokens" not in small
