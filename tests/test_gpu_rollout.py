"""Paged engine on the GPU: CUDA-graph decode equals eager decode, rollout log-probs equal the
training forward's log-probs of the same tokens."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def model():
  from tunix_b200.models.transformer import ModelConfig, Transformer
  cfg = ModelConfig(num_layers=2, vocab_size=512, embed_dim=256, hidden_dim=512, num_heads=4, head_dim=128,
                    num_kv_heads=2, use_qk_norm=True, dtype=torch.bfloat16)
  with torch.device("cuda"):
    m = Transformer(cfg)
  return m.init_weights(seed=0, scale=0.05).eval()


def test_graph_decode_matches_eager_and_training_logprobs(kernel_lib):
  from tunix_b200.ops import _lib
  from tunix_b200.rollout import EngineConfig, PagedEngine
  m = model()
  rng = np.random.default_rng(0)
  prompts = [rng.integers(3, 500, size=n).tolist() for n in (5, 37, 37, 64, 130)] + [[7, 8, 9]] * 3
  outs = []
  for graphs in (False, True):
    eng = PagedEngine(m, EngineConfig(page_size=16, max_batch=8, max_seq_len=256, use_cuda_graphs=graphs))
    outs.append(eng.generate(prompts, 24, temperature=1.0, seed=5))
    assert eng.cache.allocator.free_pages == eng.cache.num_pages
    if graphs:
      assert any(v is not False for v in eng._graphs.values()), "decode step was not captured"
  _lib.check_status()
  for a, b in zip(outs[0].tokens, outs[1].tokens):
    assert a.tolist() == b.tolist()
  # log-probs reported by the engine vs a plain forward over prompt + completion
  for p, t, lp in zip(prompts, outs[1].tokens, outs[1].logprobs):
    seq = torch.tensor([p + t.tolist()], device="cuda")
    with torch.no_grad():
      logits, _ = m(seq, None, None, None)
    ref = torch.log_softmax(logits[0, len(p) - 1:-1].float(), -1).gather(-1, seq[0, len(p):, None])[:, 0]
    np.testing.assert_allclose(lp, ref.cpu().numpy(), rtol=0, atol=0.08)
  assert len({tuple(t.tolist()) for t in outs[1].tokens[-3:]}) > 1     # samples of one prompt differ


def test_decode_of_96_sequences_matches_training_logprobs(kernel_lib):
  """Above 64 rows the plain decode products take the general GEMM (residual through accumulate), gate|up keeps
  the fused-GLU skinny kernel: same log-probs as the training forward."""
  from tunix_b200.ops import _lib
  from tunix_b200.rollout import EngineConfig, PagedEngine
  m = model()
  rng = np.random.default_rng(1)
  prompts = [rng.integers(3, 500, size=int(n)).tolist() for n in rng.integers(4, 40, size=96)]
  eng = PagedEngine(m, EngineConfig(page_size=16, max_batch=96, max_seq_len=128, use_cuda_graphs=True))
  out = eng.generate(prompts, 8, temperature=1.0, seed=3)
  _lib.check_status()
  for p, t, lp in list(zip(prompts, out.tokens, out.logprobs))[::7]:
    seq = torch.tensor([p + t.tolist()], device="cuda")
    with torch.no_grad():
      logits, _ = m(seq, None, None, None)
    ref = torch.log_softmax(logits[0, len(p) - 1:-1].float(), -1).gather(-1, seq[0, len(p):, None])[:, 0]
    np.testing.assert_allclose(lp, ref.cpu().numpy(), rtol=0, atol=0.08)
