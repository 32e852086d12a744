"""Qwen 3 / 3.5, dense and mixture-of-experts (tunix/models/qwen3/model.py:136-327): per-head
q/k RMSNorm before RoPE, RoPE theta 1e6, SwiGLU; MoE variants route each token to the top-k of
E experts with a softmax router and renormalised weights."""
from __future__ import annotations

from .._family import make_family
from ..transformer import RematConfig, Transformer  # noqa: F401

_D = dict(norm_eps=1e-6, rope_theta=1_000_000.0, activation="silu", use_qk_norm=True)


def _moe(hidden, experts, topk, **kw):
  return dict(hidden_dim=hidden, moe_hidden_dim=hidden, num_experts=experts, num_experts_per_tok=topk, **kw)


ModelConfig = make_family(
    "qwen3", _D,
    presets={
        "qwen3_0p6b": dict(num_layers=28, vocab_size=151936, embed_dim=1024, hidden_dim=3072, num_heads=16,
                           head_dim=128, num_kv_heads=8, weight_tying=True),
        "qwen3_1p7b": dict(num_layers=28, vocab_size=151936, embed_dim=2048, hidden_dim=6144, num_heads=16,
                           head_dim=128, num_kv_heads=8, weight_tying=True),
        "qwen3_4b": dict(num_layers=36, vocab_size=151936, embed_dim=2560, hidden_dim=9728, num_heads=32,
                         head_dim=128, num_kv_heads=8, weight_tying=True),
        "qwen3_4b_instruct_2507": dict(num_layers=36, vocab_size=151936, embed_dim=2560, hidden_dim=9728, num_heads=32,
                                       head_dim=128, num_kv_heads=8, weight_tying=True, rope_theta=5_000_000.0),
        "qwen3_8b": dict(num_layers=36, vocab_size=151936, embed_dim=4096, hidden_dim=12288, num_heads=32,
                         head_dim=128, num_kv_heads=8),
        "qwen3_14b": dict(num_layers=40, vocab_size=151936, embed_dim=5120, hidden_dim=17408, num_heads=40,
                          head_dim=128, num_kv_heads=8),
        "qwen3_32b": dict(num_layers=64, vocab_size=151936, embed_dim=5120, hidden_dim=25600, num_heads=64,
                          head_dim=128, num_kv_heads=8),
        "qwen3_30b_a3b": _moe(768, 128, 8, num_layers=48, vocab_size=151936, embed_dim=2048, num_heads=32,
                              head_dim=128, num_kv_heads=4),
        "qwen3p5_35b_a3b": _moe(512, 256, 8, num_layers=40, vocab_size=248320, embed_dim=2048, num_heads=16,
                                head_dim=256, num_kv_heads=2, rope_theta=10_000_000.0),
        "qwen3p5_397b_a17b": _moe(1024, 512, 10, num_layers=60, vocab_size=248320, embed_dim=4096, num_heads=32,
                                  head_dim=256, num_kv_heads=2, rope_theta=10_000_000.0),
    },
    aliases={"qwen3_0p6b_base": "qwen3_0p6b", "qwen3_1p7b_base": "qwen3_1p7b", "qwen3_4b_base": "qwen3_4b",
             "qwen3_4b_thinking_2507": "qwen3_4b_instruct_2507", "qwen3_8b_base": "qwen3_8b",
             "qwen3_14b_base": "qwen3_14b"},
)


class Qwen3(Transformer):
  """Qwen 3 decoder (dense or MoE)."""
