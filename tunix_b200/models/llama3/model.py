"""Llama 3 / 3.1 / 3.2 (tunix/models/llama3/model.py:86-189): RMSNorm `w * x / rms`,
RoPE theta 500 000, SwiGLU, GQA; 3.2 ties the output head to the embedding."""
from __future__ import annotations

from .._family import make_family
from ..transformer import RematConfig, Transformer  # noqa: F401

_D = dict(norm_eps=1e-5, rope_theta=500_000.0, activation="silu")

ModelConfig = make_family(
    "llama3", _D,
    presets={
        "llama3p2_1b": dict(num_layers=16, vocab_size=128256, embed_dim=2048, hidden_dim=8192, num_heads=32,
                            head_dim=64, num_kv_heads=8, weight_tying=True),
        "llama3p2_3b": dict(num_layers=28, vocab_size=128256, embed_dim=3072, hidden_dim=8192, num_heads=24,
                            head_dim=128, num_kv_heads=8, weight_tying=True),
        "llama3p1_8b": dict(num_layers=32, vocab_size=128256, embed_dim=4096, hidden_dim=14336, num_heads=32,
                            head_dim=128, num_kv_heads=8),
        "llama3_70b": dict(num_layers=80, vocab_size=128256, embed_dim=8192, hidden_dim=28672, num_heads=64,
                           head_dim=128, num_kv_heads=8),
        "llama3p1_405b": dict(num_layers=126, vocab_size=128256, embed_dim=16384, hidden_dim=53248, num_heads=128,
                              head_dim=128, num_kv_heads=8),
    },
    aliases={"llama3p2_1b_instruct": "llama3p2_1b", "llama3p2_3b_instruct": "llama3p2_3b",
             "llama3p1_8b_instruct": "llama3p1_8b", "llama3p1_70b": "llama3_70b", "llama3_8b": "llama3p1_8b"},
)


class Llama3(Transformer):
  """Llama 3 decoder."""
