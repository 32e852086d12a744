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
  model = Transformer(cfg, device=dev).init_weights(seed=0, scale=0.08)
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
    for x, y in zip(a.tokens, b.tokens):
      n = min(len(x), len(y))
      # greedy decoding in bf16 through two attention implementations: count until the first divergence
      k = next((i for i in range(n) if int(x[i]) != int(y[i])), n)
      same, total = same + k, total + n
    return same / max(total, 1), a

  first, out = agreement()
  assert first >= 0.8, first
  assert out.logprobs is not None and all(len(lp) == len(t) for lp, t in zip(out.logprobs, out.tokens))
  with torch.no_grad():
    for p in model.parameters():
      p.add_(0.05 * torch.randn_like(p))
  stale, _ = agreement()                      # the engine still holds the old weights
  engine.update_params(dict(model.named_parameters()))
  fresh, _ = agreement()
  assert fresh >= 0.8 and fresh >= stale, (stale, fresh)
  engine.close()
