"""Gemma 1 / 1.1 / 2 (tunix/models/gemma/model.py:91-215): embeddings scaled by sqrt(D), RMSNorm
with `(1 + w)` and eps 1e-6, GeGLU (tanh GELU), tied head, RoPE theta 10 000; Gemma 2 adds
attention-logit soft-cap 50, final soft-cap 30, alternating 4096-token sliding-window layers and
post-attention / post-FFW norms."""
from __future__ import annotations

from .._family import make_family
from ..transformer import AttentionType, RematConfig, Transformer  # noqa: F401

_D = dict(norm_eps=1e-6, rope_theta=10_000.0, activation="gelu", norm_offset=1.0, embed_scale=True,
          weight_tying=True)
_G2 = dict(final_logit_softcap=30.0, attn_logits_soft_cap=50.0, sliding_window_size=4096, use_post_attn_norm=True,
           use_post_ffw_norm=True, attention_types=(AttentionType.LOCAL_SLIDING, AttentionType.GLOBAL))

ModelConfig = make_family(
    "gemma", _D,
    presets={
        "gemma_2b": dict(num_layers=18, vocab_size=256128, embed_dim=2048, hidden_dim=16384, num_heads=8,
                         head_dim=256, num_kv_heads=1),
        "gemma_7b": dict(num_layers=28, vocab_size=256128, embed_dim=3072, hidden_dim=24576, num_heads=16,
                         head_dim=256, num_kv_heads=16),
        "gemma2_2b": dict(num_layers=26, vocab_size=256128, embed_dim=2304, hidden_dim=9216, num_heads=8,
                          head_dim=256, num_kv_heads=4, **_G2),
        "gemma2_9b": dict(num_layers=42, vocab_size=256128, embed_dim=3584, hidden_dim=28672, num_heads=16,
                          head_dim=256, num_kv_heads=8, **_G2),
    },
    aliases={"gemma_2b_it": "gemma_2b", "gemma1p1_2b_it": "gemma_2b", "gemma_7b_it": "gemma_7b",
             "gemma1p1_7b_it": "gemma_7b", "gemma2_2b_it": "gemma2_2b", "gemma2_9b_it": "gemma2_9b"},
)


class Gemma(Transformer):
  """Gemma 1 / 2 decoder."""
