"""`VllmSampler` against the real vLLM engine (not the fake of tests/test_generate_perf_utils.py): a tiny random Qwen3
starts from an exported `config.json` with dummy weights, receives this package's weights through `update_params`,
and must then decode greedily like this package's own sampler - before and after a second weight sync.

Starting a vLLM engine takes minutes on a fresh machine (kernel caches are empty), so the test runs only when
TUNIX_B200_RUN_VLLM=1."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(os.environ.get("TUNIX_B200_RUN_VLLM") != "1", reason="set TUNIX_B200_RUN_VLLM=1 (slow engine start)")
def test_real_vllm_engine_generates_with_synced_weights():
  pytest.importorskip("vllm")
  os.environ.setdefault("VLLM_USE_FLASHINFER_SAMPLER", "0")
  from tests.test_rl_grpo import ToyTokenizer
  from tunix_b200.common.configs import CacheConfig
  from tunix_b200.generate import sampler as sampler_lib, vllm_sampler as vs
  from tunix_b200.models.qwen3.model import ModelConfig
  from tunix_b200.models.transformer import Transformer
  dev = torch.device("cuda", 0)
  cfg = ModelConfig(num_layers=2, vocab_size=512, embed_dim=256, hidden_dim=512, num_heads=4, head_dim=64,
                    num_kv_heads=2, dtype=torch.bfloat16, max_position=128)
  model = Transformer(cfg, device=dev).init_weights(seed=0, scale=0.15)
  tok = ToyTokenizer(vocab=512)
  conf = vs.VllmConfig(max_model_len=128, hbm_utilization=0.08, seed=0,
                       engine_kwargs={"enforce_eager": True, "attention_backend": "TRITON_ATTN", "dtype": "bfloat16"})
  engine = vs.VllmSampler(tok, conf, model=model)
  own = sampler_lib.Sampler(model, tok, CacheConfig(cache_size=128, num_layers=2, num_kv_heads=2, head_dim=64))
  prompts = ["the quick brown fox jumps", "a b c d e f g h", "weights arrive through load_weights"]

  def agreement():
    a = engine(prompts, max_generation_steps=12, temperature=0.0, return_logprobs=True, eos_tokens=[511])
    b = own(input_strings=prompts, max_generation_steps=12, temperature=0.0, echo=False, pad_output=False,
            eos_tokens=[511], return_logprobs=True)
    same = total = 0
    gaps = []
    for x, y, lx, ly in zip(a.tokens, b.tokens, a.logprobs, b.logprobs):
      n = min(len(x), len(y))
      # greedy decoding in bf16 through two attention implementations: near-ties of a random model flip, and
      # everything after a flip differs, so only the common prefix counts
      k = next((i for i in range(n) if int(x[i]) != int(y[i])), n)
      same, total = same + k, total + n
      gaps += [abs(float(lx[i]) - float(ly[i])) for i in range(k)]
    return same / max(total, 1), float(np.mean(gaps)) if gaps else float("inf"), a

  first, gap, out = agreement()
  assert first >= 0.5 and gap < 0.15, (first, gap)      # dummy weights would agree on about 1 token in 512
  assert out.logprobs is not None and all(len(lp) == len(t) for lp, t in zip(out.logprobs, out.tokens))
  with torch.no_grad():
    for p in model.parameters():
      p.add_(0.05 * torch.randn_like(p))
  stale, _, _ = agreement()                   # the engine still holds the old weights
  engine.update_params(dict(model.named_parameters()))
  fresh, gap, _ = agreement()
  assert fresh >= 0.5 and gap < 0.15 and fresh >= stale, (stale, fresh, gap)
  print(f"vllm agreement: first {first:.2f}, stale {stale:.2f}, fresh {fresh:.2f}, logprob gap {gap:.3f}")
  # server mode on the same engine: requests go through the step-level driver (add_request / step / futures)
  import dataclasses
  served = vs.VllmSampler(tok, dataclasses.replace(conf, server_mode=True, submission_threshold=2,
                                                   submission_timeout_s=0.05), model=None, llm=engine.llm)
  assert served._step_driver is not None
  batch = engine(prompts, max_generation_steps=12, temperature=0.0, eos_tokens=[511])
  stepped = served(prompts, max_generation_steps=12, temperature=0.0, eos_tokens=[511])
  assert all(np.array_equal(x, y) for x, y in zip(batch.tokens, stepped.tokens))
  assert served._step_driver.steps >= 12 and served._step_driver.last_error is None
  served.close()
  engine.close()


@pytest.mark.skipif(os.environ.get("TUNIX_B200_RUN_VLLM") != "1", reason="set TUNIX_B200_RUN_VLLM=1 (slow engine start)")
def test_grpo_steps_with_the_vllm_rollout_engine():
  """`ClusterConfig(rollout_engine="vllm")`: the rollout role is a real vLLM engine that receives the actor's
  weights after every optimizer step; two GRPO steps run, and the engine's greedy decode follows the actor."""
  pytest.importorskip("vllm")
  os.environ.setdefault("VLLM_USE_FLASHINFER_SAMPLER", "0")
  from tests.test_rl_grpo import ToyTokenizer, prompts_ds, reward_len
  from tunix_b200 import optim
  from tunix_b200.common.configs import CacheConfig, ClusterConfig, RLTrainingConfig, Role, RolloutConfig
  from tunix_b200.generate import sampler as sampler_lib
  from tunix_b200.models.qwen3.model import ModelConfig
  from tunix_b200.models.transformer import Transformer
  from tunix_b200.rl import rl_cluster
  from tunix_b200.rl.grpo import grpo_learner
  dev = torch.device("cuda", 0)
  cfg = ModelConfig(num_layers=2, vocab_size=512, embed_dim=256, hidden_dim=512, num_heads=4, head_dim=64,
                    num_kv_heads=2, dtype=torch.bfloat16, max_position=128)
  actor = Transformer(cfg, device=dev).init_weights(seed=0, scale=0.15)
  reference = Transformer(cfg, device=dev).init_weights(seed=0, scale=0.15)
  tok = ToyTokenizer(vocab=512)
  tc = RLTrainingConfig(actor_optimizer=optim.adamw(2e-3), eval_every_n_steps=100, max_steps=2, pbar_description=None)
  rc = RolloutConfig(max_tokens_to_generate=8, max_prompt_length=8, kv_cache_size=64, temperature=1.0, top_p=1.0,
                     seed=3, return_logprobs=True, eos_tokens=[511], rollout_vllm_hbm_utilization=0.08,
                     rollout_vllm_kwargs={"enforce_eager": True, "attention_backend": "TRITON_ATTN",
                                          "dtype": "bfloat16"})
  cc = ClusterConfig(role_to_mesh={Role.ACTOR: None, Role.REFERENCE: None, Role.ROLLOUT: None},
                     rollout_engine="vllm", training_config=tc, rollout_config=rc)
  cl = rl_cluster.RLCluster(actor=actor, reference=reference, tokenizer=tok, cluster_config=cc)
  before = {n: p.detach().clone() for n, p in actor.named_parameters()}
  learner = grpo_learner.GRPOLearner(rl_cluster=cl, algo_config=grpo_learner.GRPOConfig(num_generations=2),
                                     reward_fns=[reward_len])
  learner.train(prompts_ds(2))
  assert cl.actor_trainer.train_steps == 2
  assert any(not torch.equal(p, before[n]) for n, p in actor.named_parameters())
  losses = cl._rl_metrics_logger.get_metric_history("", "loss", "train")
  assert len(losses) == 2 and all(np.isfinite(l) for l in losses)
  # after the last sync the engine decodes like the trained actor
  prompts = ["alpha beta gamma", "delta eps zeta"]
  own = sampler_lib.Sampler(actor, tok, CacheConfig(cache_size=64, num_layers=2, num_kv_heads=2, head_dim=64))
  a = cl._rollout._sampler(prompts, max_generation_steps=8, temperature=0.0, eos_tokens=[511])
  b = own(input_strings=prompts, max_generation_steps=8, temperature=0.0, echo=False, pad_output=False, eos_tokens=[511])
  first = [int(x[0]) == int(y[0]) for x, y in zip(a.tokens, b.tokens)]
  assert all(first), (a.tokens, b.tokens)
