"""Gemma 3 text decoder (tunix/models/gemma3/model.py:100-310): Gemma 2 layout plus q/k-norm,
five local sliding-window layers per global layer, separate RoPE bases for local (1e4) and
global (1e6, positions scaled by 8 from 4b up) layers, no soft-caps."""
from __future__ import annotations

from .._family import make_family
from ..transformer import AttentionType, RematConfig, Transformer  # noqa: F401

_PATTERN = (AttentionType.LOCAL_SLIDING,) * 5 + (AttentionType.GLOBAL,)
_D = dict(norm_eps=1e-6, rope_theta=1_000_000.0, local_rope_theta=10_000.0, activation="gelu", norm_offset=1.0,
          embed_scale=True, weight_tying=True, use_qk_norm=True, use_post_attn_norm=True, use_post_ffw_norm=True,
          attention_types=_PATTERN, vocab_size=262144)

ModelConfig = make_family(
    "gemma3", _D,
    presets={
        "gemma3_270m": dict(num_layers=18, embed_dim=640, hidden_dim=2048, num_heads=4, head_dim=256, num_kv_heads=1,
                            sliding_window_size=512),
        "gemma3_1b": dict(num_layers=26, embed_dim=1152, hidden_dim=6912, num_heads=4, head_dim=256, num_kv_heads=1,
                          sliding_window_size=512),
        "gemma3_4b": dict(num_layers=34, embed_dim=2560, hidden_dim=10240, num_heads=8, head_dim=256, num_kv_heads=4,
                          sliding_window_size=1024, rope_scale_factor=8.0),
        "gemma3_12b": dict(num_layers=48, embed_dim=3840, hidden_dim=15360, num_heads=16, head_dim=256,
                           num_kv_heads=8, sliding_window_size=1024, rope_scale_factor=8.0),
        "gemma3_27b": dict(num_layers=62, embed_dim=5376, hidden_dim=21504, num_heads=32, head_dim=128,
                           num_kv_heads=16, sliding_window_size=1024, rope_scale_factor=8.0,
                           query_pre_attn_scalar=5376 / 32),
    },
    aliases={"gemma3_270m_it": "gemma3_270m", "gemma3_1b_it": "gemma3_1b", "gemma3_1b_pt": "gemma3_1b",
             "gemma3_4b_it": "gemma3_4b", "gemma3_4b_pt": "gemma3_4b", "gemma3_12b_it": "gemma3_12b",
             "gemma3_12b_pt": "gemma3_12b", "gemma3_27b_it": "gemma3_27b", "gemma3_27b_pt": "gemma3_27b"},
)


class Gemma3(Transformer):
  """Gemma 3 text decoder."""
