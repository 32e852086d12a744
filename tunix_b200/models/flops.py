"""FLOP accounting from a model configuration (no tracing, no cost analysis)."""
from __future__ import annotations

from .transformer import ModelConfig, num_params


def matmul_params(cfg: ModelConfig) -> int:
  """Parameters that take part in matrix multiplications for one token (active experts only);
  the embedding gather is excluded, the output head is included."""
  D, N, K, H, V, L = cfg.embed_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.vocab_size, cfg.num_layers
  attn = D * (N + 2 * K) * H + N * H * D
  if cfg.is_moe:
    mlp = D * cfg.num_experts + cfg.num_experts_per_tok * 3 * D * cfg.moe_hidden_dim
  else:
    mlp = 3 * D * cfg.hidden_dim
  return L * (attn + mlp) + V * D


def forward_flops_per_token(cfg: ModelConfig, seq_len: int, causal: bool = True) -> float:
  attn = 4.0 * cfg.num_layers * cfg.num_heads * cfg.head_dim * seq_len * (0.5 if causal else 1.0)
  return 2.0 * matmul_params(cfg) + attn


def train_flops_per_token(cfg: ModelConfig, seq_len: int, causal: bool = True) -> float:
  """Forward + backward (3x forward); recomputation is not counted as useful work."""
  return 3.0 * forward_flops_per_token(cfg, seq_len, causal)
