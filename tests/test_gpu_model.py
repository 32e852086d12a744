"""End-to-end numerics on the GPU: the bf16 kernel path of the decoder against the fp32 PyTorch
statement of the same model (forward logits, loss and parameter gradients)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _models(family_cfg, **kw):
  from tunix_b200.models.transformer import Transformer
  cfg32 = family_cfg(dtype=torch.float32, **kw)
  ref = Transformer(cfg32).init_weights(seed=3)
  cfg16 = cfg32.replace(dtype=torch.bfloat16)
  gpu = Transformer(cfg16, device="cuda")
  with torch.no_grad():
    for (n, p), (_, q) in zip(ref.named_parameters(), gpu.named_parameters()):
      q.copy_(p.to(torch.bfloat16))
      p.copy_(q.float().cpu())      # the oracle sees the bf16-rounded weights
  return ref, gpu


@pytest.mark.parametrize("family", ["llama3", "qwen3", "gemma"])
def test_forward_backward_matches_fp32_oracle(kernel_lib, family):
  import importlib
  from tunix_b200.ops import _lib
  from tunix_b200.sft.peft_trainer import _default_loss_fn
  mod = importlib.import_module(f"tunix_b200.models.{family}.model")
  ref, gpu = _models(mod.ModelConfig, num_layers=2, vocab_size=1024, embed_dim=256, hidden_dim=512, num_heads=4,
                     head_dim=64, num_kv_heads=2)
  torch.manual_seed(0)
  tok = torch.randint(0, 1024, (2, 128))
  mask = torch.ones(2, 128)
  mask[:, :32] = 0
  lo_ref = _default_loss_fn(ref, tok, mask)
  lo_gpu = _default_loss_fn(gpu, tok.cuda(), mask.cuda())
  l_ref = lo_ref.primary_loss.compute()
  l_gpu = lo_gpu.primary_loss.compute()
  assert abs(l_ref.item() - l_gpu.item()) < 3e-2 * max(1.0, abs(l_ref.item())), (l_ref.item(), l_gpu.item())
  lo_ref.primary_loss.unreduced_sum.backward()
  lo_gpu.primary_loss.unreduced_sum.backward()
  _lib.check_status()
  bad = []
  for (n, p), (_, q) in zip(ref.named_parameters(), gpu.named_parameters()):
    g_ref = p.grad
    g_gpu = q.grad.float().cpu()
    rel = (g_ref - g_gpu).norm() / (g_ref.norm() + 1e-6)
    if rel > 0.08:
      bad.append((n, rel.item()))
  assert not bad, bad
  with torch.no_grad():
    lg_ref, _ = ref(tok)
    lg_gpu, _ = gpu(tok.cuda())
  rel = (lg_ref - lg_gpu.float().cpu()).norm() / lg_ref.norm()
  assert rel < 3e-2, rel


def test_trainer_step_on_gpu(kernel_lib):
  import __graft_entry__ as ge
  ge.smoke()
