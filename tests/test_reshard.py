"""Layout transfer of parameter trees on CPU: same-shape copies and tensor-parallel slices."""
import pytest
import torch

from tunix_b200.dist import tp as tp_lib, weight_sync
from tunix_b200.models.llama3 import model as llama
from tunix_b200.models.transformer import Transformer
from tunix_b200.rl import reshard


def _tiny():
  cfg = llama.ModelConfig.llama3p2_1b()
  cfg.num_layers, cfg.vocab_size, cfg.embed_dim, cfg.hidden_dim = 1, 64, 64, 128
  cfg.num_heads, cfg.num_kv_heads, cfg.head_dim = 4, 2, 16
  return cfg


def test_same_shape_leaves_are_cast_and_aliases_pass_through():
  a = {"x": torch.randn(4, 4), "y": torch.randn(3)}
  t = {"x": torch.empty(4, 4, dtype=torch.bfloat16), "y": a["y"]}
  out = reshard.reshard_pytree(a, t)
  assert out["x"].dtype == torch.bfloat16 and torch.equal(out["x"], a["x"].bfloat16())
  assert out["y"] is a["y"]
  with pytest.raises(ValueError):
    reshard.reshard_pytree({"x": torch.randn(4, 4)}, {"x": torch.empty(2, 4)})


@pytest.mark.parametrize("tp", [2, 4])
def test_tensor_parallel_targets_are_cut_with_the_transfer_kernels_block_table(tp):
  torch.manual_seed(0)
  cfg = _tiny()
  full = Transformer(cfg)
  source = {n: torch.randn(p.shape) for n, p in full.named_parameters()}
  for r in range(tp):
    target = {}
    for n, p in source.items():
      shape, _ = weight_sync.tp_blocks(n, p.shape, cfg, tp, r)
      target[n] = torch.empty(shape, dtype=torch.float32)
    out = reshard.reshard_pytree(source, target, model_config=cfg, tp=tp, tp_rank=r)
    H, N, K, F = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads, cfg.hidden_dim
    qkv = source["layers.0.attn.qkv_proj.w"]
    nq = N // tp * H
    kv_idx = r * K // tp if K >= tp else r // (tp // K)
    kvl = max(1, K // tp) * H
    want = torch.cat([qkv[r * nq:(r + 1) * nq], qkv[N * H + kv_idx * kvl:N * H + (kv_idx + 1) * kvl],
                      qkv[(N + K) * H + kv_idx * kvl:(N + K) * H + (kv_idx + 1) * kvl]])
    assert torch.equal(out["layers.0.attn.qkv_proj.w"], want)
    down = source["layers.0.mlp.down_proj.w"]
    assert torch.equal(out["layers.0.mlp.down_proj.w"], down[:, r * (F // tp):(r + 1) * (F // tp)])
    assert torch.equal(out["layers.0.input_layernorm.w"], source["layers.0.input_layernorm.w"])
