"""Qwen 2.5 and DeepSeek-R1-distill-Qwen (tunix/models/qwen2/model.py:97-238): like Llama with
biases on q/k/v, RoPE theta 1e6, tied embeddings on the small sizes."""
from __future__ import annotations

from .._family import make_family
from ..transformer import RematConfig, Transformer  # noqa: F401

_D = dict(norm_eps=1e-6, rope_theta=1_000_000.0, activation="silu", qkv_bias=True)

ModelConfig = make_family(
    "qwen2", _D,
    presets={
        "qwen2p5_0p5b": dict(num_layers=24, vocab_size=151936, embed_dim=896, hidden_dim=4864, num_heads=14,
                             head_dim=64, num_kv_heads=2, weight_tying=True),
        "deepseek_r1_distill_qwen_1p5b": dict(num_layers=28, vocab_size=151936, embed_dim=1536, hidden_dim=8960,
                                              num_heads=12, head_dim=128, num_kv_heads=2, rope_theta=10000.0),
        "qwen2p5_1p5b": dict(num_layers=28, vocab_size=151936, embed_dim=1536, hidden_dim=8960, num_heads=12,
                             head_dim=128, num_kv_heads=2, weight_tying=True),
        "qwen2p5_math_1p5b": dict(num_layers=28, vocab_size=151936, embed_dim=1536, hidden_dim=8960, num_heads=12,
                                  head_dim=128, num_kv_heads=2, rope_theta=10000.0, weight_tying=True),
        "qwen2p5_3b": dict(num_layers=36, vocab_size=151936, embed_dim=2048, hidden_dim=11008, num_heads=16,
                           head_dim=128, num_kv_heads=2, weight_tying=True),
        "qwen2p5_7b": dict(num_layers=28, vocab_size=152064, embed_dim=3584, hidden_dim=18944, num_heads=28,
                           head_dim=128, num_kv_heads=4),
    },
    aliases={"qwen2p5_0p5b_instruct": "qwen2p5_0p5b", "qwen2p5_coder_0p5b": "qwen2p5_0p5b",
             "qwen2p5_1p5b_instruct": "qwen2p5_1p5b", "qwen2p5_3b_instruct": "qwen2p5_3b",
             "qwen2p5_coder_3b": "qwen2p5_3b", "qwen2p5_7b_instruct": "qwen2p5_7b", "qwen2p5_coder_7b": "qwen2p5_7b"},
)


class Qwen2(Transformer):
  """Qwen 2.5 decoder."""
