"""Gemma 4 checkpoints in the Hugging Face safetensors naming <-> this package's parameters
(tunix/models/gemma4/params_safetensors.py:27-863).

The checkpoint stores torch `Linear` weights as [out, in], which is also how this package keeps every projection,
so - unlike the reference, which re-lays everything out for einsum - importing is renaming plus a few *fusions*:

  text        gate_proj | up_proj            -> mlp.gate_up_proj          (rows: gate then up)
  vision      q_proj | k_proj | v_proj       -> attn.qkv_proj.w           (rows: q, k, v); clamps per segment, the
              gate_proj | up_proj            -> mlp.gate_up_proj.w         k clamps also serve v, the gate clamps up
              position_embedding_table [2, S, D] -> pos_emb [S, 2, D]
  audio       q / k / v projections stay apart (`attn.qkv.{0,1,2}`), clamps map one to one

The table below is written once, as (checkpoint key pattern, parameter name pattern) pairs with `{i}` for a layer
index; `from_hf` and `to_hf` are generated from it, so the two directions cannot drift apart. Checkpoint keys
may carry the `model.language_model.` / `model.` prefixes or not.
"""
from __future__ import annotations

import os
import re
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Tuple

import torch

_TEXT_PREFIXES = ("model.language_model.", "language_model.model.", "model.", "")
_TOWER_PREFIXES = ("model.", "")
_CLAMPS = (("input_min", "clip_input_min"), ("input_max", "clip_input_max"),
           ("output_min", "clip_output_min"), ("output_max", "clip_output_max"))

# (checkpoint key, parameter name); {i} = layer index. One-to-one renames.
_TEXT = [
    ("embed_tokens.weight", "embedder.input_embedding"),
    ("embed_tokens_per_layer.weight", "embedder.per_layer_input_embedding"),
    ("per_layer_model_projection.weight", "embedder.per_layer_model_projection"),
    ("per_layer_projection_norm.weight", "embedder.per_layer_projection_norm"),
    ("norm.weight", "final_norm"),
    ("layers.{i}.input_layernorm.weight", "layers.{i}.pre_attention_norm"),
    ("layers.{i}.post_attention_layernorm.weight", "layers.{i}.post_attention_norm"),
    ("layers.{i}.pre_feedforward_layernorm.weight", "layers.{i}.pre_ffw_norm"),
    ("layers.{i}.post_feedforward_layernorm.weight", "layers.{i}.post_ffw_norm"),
    ("layers.{i}.post_feedforward_layernorm_1.weight", "layers.{i}.dense_post_ffw_norm"),
    ("layers.{i}.pre_feedforward_layernorm_2.weight", "layers.{i}.moe_pre_ffw_norm"),
    ("layers.{i}.post_feedforward_layernorm_2.weight", "layers.{i}.moe_post_ffw_norm"),
    ("layers.{i}.layer_scalar", "layers.{i}.skip_scale"),
    ("layers.{i}.per_layer_input_gate.weight", "layers.{i}.per_layer_input_gate"),
    ("layers.{i}.per_layer_projection.weight", "layers.{i}.per_layer_projection"),
    ("layers.{i}.post_per_layer_input_norm.weight", "layers.{i}.post_per_layer_input_norm"),
    ("layers.{i}.self_attn.q_proj.weight", "layers.{i}.attn.q_proj"),
    ("layers.{i}.self_attn.k_proj.weight", "layers.{i}.attn.k_proj"),
    ("layers.{i}.self_attn.v_proj.weight", "layers.{i}.attn.v_proj"),
    ("layers.{i}.self_attn.o_proj.weight", "layers.{i}.attn.o_proj"),
    ("layers.{i}.self_attn.q_norm.weight", "layers.{i}.attn.q_norm"),
    ("layers.{i}.self_attn.k_norm.weight", "layers.{i}.attn.k_norm"),
    ("layers.{i}.mlp.down_proj.weight", "layers.{i}.mlp.down_proj"),
    ("layers.{i}.router.proj.weight", "layers.{i}.moe.router"),
    ("layers.{i}.router.scale", "layers.{i}.moe.router_scale"),
    ("layers.{i}.router.per_expert_scale", "layers.{i}.moe.per_expert_scale"),
    ("layers.{i}.experts.gate_up_proj", "layers.{i}.moe.gate_up_proj"),
    ("layers.{i}.experts.down_proj", "layers.{i}.moe.down_proj"),
]
_VISION = [
    ("vision_tower.patch_embedder.input_proj.weight", "vision_encoder.input_projection"),
    ("vision_tower.std_scale", "vision_encoder.std_scale"),
    ("vision_tower.std_bias", "vision_encoder.std_bias"),
    ("vision_tower.encoder.layers.{i}.input_layernorm.weight", "vision_encoder.layers.{i}.pre_attention_norm"),
    ("vision_tower.encoder.layers.{i}.post_attention_layernorm.weight", "vision_encoder.layers.{i}.post_attention_norm"),
    ("vision_tower.encoder.layers.{i}.pre_feedforward_layernorm.weight", "vision_encoder.layers.{i}.pre_ffw_norm"),
    ("vision_tower.encoder.layers.{i}.post_feedforward_layernorm.weight", "vision_encoder.layers.{i}.post_ffw_norm"),
    ("vision_tower.encoder.layers.{i}.self_attn.q_norm.weight", "vision_encoder.layers.{i}.attn.query_norm"),
    ("vision_tower.encoder.layers.{i}.self_attn.k_norm.weight", "vision_encoder.layers.{i}.attn.key_norm"),
]
_AUDIO = [
    ("audio_tower.subsample_conv_projection.layer0.conv.weight", "audio_encoder.feature.conv0"),
    ("audio_tower.subsample_conv_projection.layer0.norm.weight", "audio_encoder.feature.norm0"),
    ("audio_tower.subsample_conv_projection.layer1.conv.weight", "audio_encoder.feature.conv1"),
    ("audio_tower.subsample_conv_projection.layer1.norm.weight", "audio_encoder.feature.norm1"),
    ("audio_tower.subsample_conv_projection.input_proj_linear.weight", "audio_encoder.feature.input_proj"),
    ("audio_tower.output_proj.weight", "audio_encoder.output_w"),
    ("audio_tower.output_proj.bias", "audio_encoder.output_b"),
    ("audio_tower.layers.{i}.norm_pre_attn.weight", "audio_encoder.conformer_layers.{i}.attn_pre_norm"),
    ("audio_tower.layers.{i}.norm_post_attn.weight", "audio_encoder.conformer_layers.{i}.attn_post_norm"),
    ("audio_tower.layers.{i}.norm_out.weight", "audio_encoder.conformer_layers.{i}.final_norm"),
    ("audio_tower.layers.{i}.self_attn.per_dim_scale", "audio_encoder.conformer_layers.{i}.attn.per_dim_scale"),
    ("audio_tower.layers.{i}.self_attn.relative_k_proj.weight", "audio_encoder.conformer_layers.{i}.attn.pos_proj"),
    ("audio_tower.layers.{i}.lconv1d.pre_layer_norm.weight", "audio_encoder.conformer_layers.{i}.lconv.pre_norm"),
    ("audio_tower.layers.{i}.lconv1d.conv_norm.weight", "audio_encoder.conformer_layers.{i}.lconv.conv_norm"),
    ("audio_tower.layers.{i}.lconv1d.depthwise_conv1d.weight", "audio_encoder.conformer_layers.{i}.lconv.depthwise"),
]
for _hf_ffn, _ours_ffn in (("feed_forward1", "ffn_start"), ("feed_forward2", "ffn_end")):
  _AUDIO += [(f"audio_tower.layers.{{i}}.{_hf_ffn}.pre_layer_norm.weight",
              f"audio_encoder.conformer_layers.{{i}}.{_ours_ffn}.pre_norm"),
             (f"audio_tower.layers.{{i}}.{_hf_ffn}.post_layer_norm.weight",
              f"audio_encoder.conformer_layers.{{i}}.{_ours_ffn}.post_norm")]
# audio linears with clamps: (checkpoint module, our module)
_AUDIO_CLIPPED = [("feed_forward1.ffw_layer_1", "ffn_start.up"), ("feed_forward1.ffw_layer_2", "ffn_start.down"),
                  ("feed_forward2.ffw_layer_1", "ffn_end.up"), ("feed_forward2.ffw_layer_2", "ffn_end.down"),
                  ("self_attn.q_proj", "attn.qkv.0"), ("self_attn.k_proj", "attn.qkv.1"), ("self_attn.v_proj", "attn.qkv.2"),
                  ("self_attn.post", "attn_out"), ("lconv1d.linear_start", "lconv.linear_start"),
                  ("lconv1d.linear_end", "lconv.linear_end")]
# vision fused linears: our module -> checkpoint modules of its segments, and which of them provides the clamps
_VISION_FUSED = [("attn.qkv_proj", ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"), (0, 1, 1)),
                 ("attn.o_proj", ("self_attn.o_proj",), (0,)),
                 ("mlp.gate_up_proj", ("mlp.gate_proj", "mlp.up_proj"), (0, 0)),
                 ("mlp.down_proj", ("mlp.down_proj",), (0,))]


class _Checkpoint:
  """Checkpoint tensors by key, tolerant of the optional prefixes and of `x.weight` vs `x.linear.weight`."""

  def __init__(self, tensors: Mapping[str, torch.Tensor]):
    self.t = tensors
    self.used: set = set()

  def find(self, key: str, prefixes: Iterable[str]) -> Optional[str]:
    variants = [key]
    if key.endswith(".weight"):
      variants.append(key[:-len(".weight")] + ".linear.weight")
      variants.append(key[:-len(".weight")])
    else:
      variants.append(key + ".weight")
    for p in prefixes:
      for v in variants:
        if p + v in self.t:
          return p + v
    return None

  def get(self, key: str, prefixes: Iterable[str]) -> Optional[torch.Tensor]:
    k = self.find(key, prefixes)
    if k is None:
      return None
    self.used.add(k)
    return self.t[k]


def _layer_counts(cfg) -> Dict[str, int]:
  return {"text": cfg.num_layers, "vision": cfg.vision_encoder.num_layers if cfg.vision_encoder is not None else 0,
          "audio": cfg.audio_encoder.num_layers if cfg.audio_encoder is not None else 0}


def _expand(table, n_layers: int):
  for hf, ours in table:
    if "{i}" in hf:
      for i in range(n_layers):
        yield hf.format(i=i), ours.format(i=i)
    else:
      yield hf, ours


def from_hf(cfg, tensors: Mapping[str, torch.Tensor], wanted: Iterable[str]) -> Dict[str, torch.Tensor]:
  """Checkpoint tensors -> {our parameter / buffer name: tensor} for the names in `wanted` (a model's state-dict
  keys). Names the checkpoint has nothing for are reported together."""
  ck = _Checkpoint(tensors)
  wanted = list(wanted)
  want = set(wanted)
  out: Dict[str, torch.Tensor] = {}
  n = _layer_counts(cfg)

  for hf, ours in _expand(_TEXT, n["text"]):
    if ours in want:
      t = ck.get(hf, _TEXT_PREFIXES)
      if t is not None:
        out[ours] = t
  for i in range(n["text"]):                                  # dense MLP: gate | up fused
    ours = f"layers.{i}.mlp.gate_up_proj"
    gate = ck.get(f"layers.{i}.mlp.gate_proj.weight", _TEXT_PREFIXES)
    up = ck.get(f"layers.{i}.mlp.up_proj.weight", _TEXT_PREFIXES)
    if ours in want and gate is not None and up is not None:
      out[ours] = torch.cat((gate, up), dim=0)
  for ours, hf in (("embedder.mm_input_projection", "embed_vision.embedding_projection.weight"),
                   ("embedder.audio_input_projection", "embed_audio.embedding_projection.weight")):
    if ours in want:
      t = ck.get(hf, _TOWER_PREFIXES)
      if t is not None:
        out[ours] = t

  if n["vision"]:
    for hf, ours in _expand(_VISION, n["vision"]):
      if ours in want:
        t = ck.get(hf, _TOWER_PREFIXES)
        if t is not None:
          out[ours] = t
    table = ck.get("vision_tower.patch_embedder.position_embedding_table", _TOWER_PREFIXES)
    if table is not None:
      out["vision_encoder.pos_emb"] = table.permute(1, 0, 2).contiguous()
    for i in range(n["vision"]):
      for ours_mod, hf_mods, clamp_from in _VISION_FUSED:
        base = f"vision_encoder.layers.{i}.{ours_mod}"
        parts = [ck.get(f"vision_tower.encoder.layers.{i}.{m}.weight", _TOWER_PREFIXES) for m in hf_mods]
        if all(p is not None for p in parts):
          out[f"{base}.w"] = torch.cat(parts, dim=0)
        for hf_name, our_name in _CLAMPS:
          if f"{base}.{our_name}" not in want:
            continue
          vals = [ck.get(f"vision_tower.encoder.layers.{i}.{hf_mods[src]}.{hf_name}", _TOWER_PREFIXES) for src in clamp_from]
          if all(v is not None for v in vals):
            out[f"{base}.{our_name}"] = torch.stack([v.reshape(()).float() for v in vals])

  if n["audio"]:
    for hf, ours in _expand(_AUDIO, n["audio"]):
      if ours in want:
        t = ck.get(hf, _TOWER_PREFIXES)
        if t is not None:
          out[ours] = t
    for i in range(n["audio"]):
      for hf_mod, ours_mod in _AUDIO_CLIPPED:
        base = f"audio_encoder.conformer_layers.{i}.{ours_mod}"
        w = ck.get(f"audio_tower.layers.{i}.{hf_mod}.weight", _TOWER_PREFIXES)
        if w is not None:
          out[f"{base}.w"] = w
        for hf_name, our_name in _CLAMPS:
          v = ck.get(f"audio_tower.layers.{i}.{hf_mod}.{hf_name}", _TOWER_PREFIXES)
          if v is not None and f"{base}.{our_name}" in want:
            out[f"{base}.{our_name}"] = v.reshape(()).float()

  missing = [k for k in wanted if k not in out]
  if missing:
    raise KeyError(f"checkpoint has nothing for {len(missing)} parameters, e.g. {missing[:6]}")
  return out


def to_hf(cfg, state: Mapping[str, torch.Tensor], prefix_text: str = "model.language_model.",
          prefix_tower: str = "model.") -> Dict[str, torch.Tensor]:
  """{our name: tensor} -> checkpoint tensors (the inverse of `from_hf`; fused weights are split again)."""
  out: Dict[str, torch.Tensor] = {}
  n = _layer_counts(cfg)
  for hf, ours in _expand(_TEXT, n["text"]):
    if ours in state:
      out[prefix_text + hf] = state[ours]
  for i in range(n["text"]):
    fused = state.get(f"layers.{i}.mlp.gate_up_proj")
    if fused is not None:
      gate, up = fused.chunk(2, dim=0)
      out[f"{prefix_text}layers.{i}.mlp.gate_proj.weight"] = gate.contiguous()
      out[f"{prefix_text}layers.{i}.mlp.up_proj.weight"] = up.contiguous()
  for ours, hf in (("embedder.mm_input_projection", "embed_vision.embedding_projection.weight"),
                   ("embedder.audio_input_projection", "embed_audio.embedding_projection.weight")):
    if ours in state:
      out[prefix_tower + hf] = state[ours]
  if n["vision"]:
    for hf, ours in _expand(_VISION, n["vision"]):
      if ours in state:
        out[prefix_tower + hf] = state[ours]
    out[prefix_tower + "vision_tower.patch_embedder.position_embedding_table"] = \
        state["vision_encoder.pos_emb"].permute(1, 0, 2).contiguous()
    for i in range(n["vision"]):
      for ours_mod, hf_mods, clamp_from in _VISION_FUSED:
        base = f"vision_encoder.layers.{i}.{ours_mod}"
        pieces = state[f"{base}.w"].chunk(len(hf_mods), dim=0)
        leaf = "linear.weight" if cfg.vision_encoder.use_clipped_linears else "weight"
        for m, piece in zip(hf_mods, pieces):
          out[f"{prefix_tower}vision_tower.encoder.layers.{i}.{m}.{leaf}"] = piece.contiguous()
        for hf_name, our_name in _CLAMPS:
          bounds = state.get(f"{base}.{our_name}")
          if bounds is None:
            continue
          for src in sorted(set(clamp_from)):                      # one clamp set per providing module
            out[f"{prefix_tower}vision_tower.encoder.layers.{i}.{hf_mods[src]}.{hf_name}"] = \
                bounds[clamp_from.index(src)].clone()
  if n["audio"]:
    for hf, ours in _expand(_AUDIO, n["audio"]):
      if ours in state:
        out[prefix_tower + hf] = state[ours]
    for i in range(n["audio"]):
      for hf_mod, ours_mod in _AUDIO_CLIPPED:
        base = f"audio_encoder.conformer_layers.{i}.{ours_mod}"
        out[f"{prefix_tower}audio_tower.layers.{i}.{hf_mod}.linear.weight"] = state[f"{base}.w"]
        for hf_name, our_name in _CLAMPS:
          out[f"{prefix_tower}audio_tower.layers.{i}.{hf_mod}.{hf_name}"] = state[f"{base}.{our_name}"].clone()
  return out


def load_checkpoint(model: torch.nn.Module, file_dir: str, strict: bool = True) -> torch.nn.Module:
  """Fills `model` (a `Gemma4`) from the `*.safetensors` files of a local checkpoint directory."""
  from .. import safetensors_io
  tensors: Dict[str, torch.Tensor] = {}
  for path in safetensors_io.list_files(file_dir):
    tensors.update(dict(safetensors_io.iter_tensors(path)))
  own = model.state_dict()
  mapped = from_hf(model.config, tensors, own.keys())
  with torch.no_grad():
    for name, value in mapped.items():
      if tuple(value.shape) != tuple(own[name].shape):
        raise ValueError(f"{name}: checkpoint shape {tuple(value.shape)} != model shape {tuple(own[name].shape)}")
      own[name].copy_(value.to(own[name].dtype))
  del strict
  return model


def save_checkpoint(model: torch.nn.Module, file_dir: str) -> str:
  """Writes `file_dir/model.safetensors` under checkpoint names."""
  from .. import safetensors_io
  os.makedirs(file_dir, exist_ok=True)
  path = os.path.join(file_dir, "model.safetensors")
  safetensors_io.save_file({k: v.detach().cpu().contiguous() for k, v in to_hf(model.config, model.state_dict()).items()},
                           path, metadata={"format": "pt"})
  return path
