"""Weight-name mappings from trainer parameters to an external engine's (Hugging Face) names.

`MappingConfig` carries what a weight-sync path needs (tunix/generate/mappings.py:70-170):
`to_hf_mappings` {own name pattern: (HF name pattern, split spec)}, the LoRA variant, per-key
hook functions, transpose axes and an optional whole-state preprocessing step. Our layers are
stored `[out, in]` like Hugging Face's, so no transposes are needed; the fused projections
(`qkv_proj`, `gate_up_proj`) map to several HF tensors, which the split spec describes as
(dimension, section sizes or number of equal chunks).

`MappingConfig.build(mapping_obj=..., model=..., backend=...)` accepts a ready config, a dict,
any object with those attributes (values may be zero-argument callables), or derives everything
from the model. `apply(config, state)` turns an own-name state dict into HF names.
"""
from __future__ import annotations

import dataclasses
import importlib
import re
from typing import Any, Callable, Dict, Optional, Tuple

import torch

KEYS = ("to_hf_mappings", "lora_to_hf_mappings", "to_hf_hook_fns", "to_hf_transpose_keys",
        "lora_to_hf_transpose_keys", "preprocess_src_state")


class BackendMappingMixin:
  """For model classes that publish per-backend mappings in their package's `BACKEND_MAPPINGS`."""

  DEFAULT_BACKEND = "vllm"
  BACKEND_PACKAGE_PATH: Optional[str] = None

  @classmethod
  def _backend_registry(cls) -> Dict[str, Any]:
    module = cls.BACKEND_PACKAGE_PATH or cls.__module__
    package = importlib.import_module(module.rsplit(".", 1)[0] if "." in module else module)
    return getattr(package, "BACKEND_MAPPINGS", {})

  @classmethod
  def mapping_for(cls, backend: Optional[str] = None) -> Dict[str, Any]:
    backend = backend or cls.DEFAULT_BACKEND
    reg = cls._backend_registry()
    if backend not in reg:
      raise RuntimeError(f"{backend} mappings not available for {cls.__name__}.")
    return reg[backend]

  @classmethod
  def to_hf_mappings(cls, backend: Optional[str] = None):
    m = cls.mapping_for(backend).get("to_hf_mappings")
    if m is None:
      raise RuntimeError(f"{backend} to_hf_mappings missing for {cls.__name__}.")
    return m

  @classmethod
  def lora_to_hf_mappings(cls, backend: Optional[str] = None):
    return cls.mapping_for(backend).get("lora_to_hf_mappings")

  @classmethod
  def to_hf_transpose_keys(cls, backend: Optional[str] = None):
    return cls.mapping_for(backend).get("to_hf_transpose_keys") or None

  @classmethod
  def lora_to_hf_transpose_keys(cls, backend: Optional[str] = None):
    return cls.mapping_for(backend).get("lora_to_hf_transpose_keys") or None

  @classmethod
  def to_hf_hook_fns(cls, backend: Optional[str] = None):
    return cls.mapping_for(backend).get("to_hf_hook_fns")

  @classmethod
  def preprocess_src_state(cls, backend: Optional[str] = None):
    return cls.mapping_for(backend).get("preprocess_src_state")


def decoder_to_hf_mappings(cfg) -> Dict[str, Tuple[Any, Any]]:
  """The mapping of `models.transformer.Transformer` for a model config: `*` stands for the layer
  index (and, in expert weights, a second `*` for the expert index on the HF side only)."""
  N, K, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
  gemma = str(getattr(cfg, "family", "")).startswith("gemma")
  L = "model.layers.*."
  m: Dict[str, Tuple[Any, Any]] = {
      "embedder.input_embedding": ("model.embed_tokens.weight", None),
      "final_norm.w": ("model.norm.weight", None),
      "lm_head.w": ("lm_head.weight", None),
      "layers.*.attn.qkv_proj.w": ((L + "self_attn.q_proj.weight", L + "self_attn.k_proj.weight",
                                    L + "self_attn.v_proj.weight"), (0, (N * H, K * H, K * H))),
      "layers.*.attn.qkv_proj.b": ((L + "self_attn.q_proj.bias", L + "self_attn.k_proj.bias",
                                    L + "self_attn.v_proj.bias"), (0, (N * H, K * H, K * H))),
      "layers.*.attn.o_proj.w": (L + "self_attn.o_proj.weight", None),
      "layers.*.attn.q_norm.w": (L + "self_attn.q_norm.weight", None),
      "layers.*.attn.k_norm.w": (L + "self_attn.k_norm.weight", None),
      "layers.*.input_layernorm.w": (L + "input_layernorm.weight", None),
      "layers.*.post_attention_layernorm.w": (
          L + ("pre_feedforward_layernorm.weight" if gemma and getattr(cfg, "use_post_attn_norm", False)
               else "post_attention_layernorm.weight"), None),
      "layers.*.post_attn_norm.w": (L + "post_attention_layernorm.weight", None),
      "layers.*.post_ffw_norm.w": (L + "post_feedforward_layernorm.weight", None),
      "layers.*.mlp.gate_up_proj.w": ((L + "mlp.gate_proj.weight", L + "mlp.up_proj.weight"), (0, 2)),
      "layers.*.mlp.down_proj.w": (L + "mlp.down_proj.weight", None),
      "layers.*.mlp.router.w": (L + "mlp.gate.weight", None),
      "layers.*.mlp.gate_up_proj": ((L + "mlp.experts.*.gate_proj.weight", L + "mlp.experts.*.up_proj.weight"),
                                    ("experts", (1, 2))),
      "layers.*.mlp.down_proj": (L + "mlp.experts.*.down_proj.weight", ("experts", None)),
  }
  return m


def decoder_lora_to_hf_mappings(cfg) -> Dict[str, Tuple[Any, Any]]:
  """LoRA factors `lora_a.<target>` [r, in] / `lora_b.<target>` [out_slice, r] under PEFT's names."""
  L = "base_model.model.model.layers.*."
  out = {}
  for own, hf in (("attn.qkv_proj", "self_attn"), ("attn.o_proj", "self_attn.o_proj"),
                  ("mlp.gate_up_proj", "mlp"), ("mlp.down_proj", "mlp.down_proj")):
    for ab, AB in (("lora_a", "lora_A"), ("lora_b", "lora_B")):
      out[f"layers.*.{own}.{ab}.*"] = (f"{L}{hf}.*.{AB}.weight" if own in ("attn.qkv_proj", "mlp.gate_up_proj")
                                       else f"{L}{hf}.{AB}.weight", None)
  return out


@dataclasses.dataclass
class MappingConfig:
  to_hf_mappings: Optional[Dict[str, Any]] = None
  lora_to_hf_mappings: Optional[Dict[str, Any]] = None
  to_hf_hook_fns: Optional[Dict[str, Any]] = None
  to_hf_transpose_keys: Optional[Dict[str, Tuple[int, ...]]] = None
  lora_to_hf_transpose_keys: Optional[Dict[str, Tuple[int, ...]]] = None
  preprocess_src_state: Optional[Callable[[Any], Any]] = None

  @classmethod
  def build(cls, mapping_obj: Any = None, model: Any = None, backend: Optional[str] = None) -> "MappingConfig":
    if mapping_obj is None and model is None:
      raise ValueError("Either mapping_obj or model must be provided (both cannot be None)")
    if isinstance(mapping_obj, cls):
      return mapping_obj
    if mapping_obj is None:
      return cls.from_model(model, backend or BackendMappingMixin.DEFAULT_BACKEND)
    values = dict(mapping_obj) if isinstance(mapping_obj, dict) else {
        k: getattr(mapping_obj, k) for k in KEYS if hasattr(mapping_obj, k)}
    resolved = {}
    for k in KEYS:
      v = values.get(k)
      if callable(v) and k != "preprocess_src_state":
        try:
          v = v()
        except TypeError:
          pass
      resolved[k] = v
    return cls(**resolved)

  @classmethod
  def from_model(cls, model: Any, backend: str = "vllm", **overrides: Any) -> "MappingConfig":
    def maybe_call(attr: str):
      v = getattr(model, attr, None)
      if v is None:
        return None
      if callable(v) and attr != "preprocess_src_state":
        try:
          return v(backend)
        except TypeError:
          return v()
      return v
    vals = {k: maybe_call(k) for k in KEYS}
    cfg = getattr(model, "config", None)
    if vals["to_hf_mappings"] is None and cfg is not None and hasattr(cfg, "num_kv_heads"):
      vals["to_hf_mappings"] = decoder_to_hf_mappings(cfg)
      vals["lora_to_hf_mappings"] = vals["lora_to_hf_mappings"] or decoder_lora_to_hf_mappings(cfg)
    vals.update(overrides)
    return cls(**vals)


def _match(pattern: str, name: str):
  rx = "^" + re.escape(pattern).replace(r"\*", r"([^.]+)") + "$"
  m = re.match(rx, name)
  return m.groups() if m else None


def _fill(pattern: str, groups) -> str:
  out = pattern
  for g in groups:
    out = out.replace("*", str(g), 1)
  return out


def apply(config: MappingConfig, state: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
  """Renames (and splits) an own-name state dict into the external names of `to_hf_mappings`.
  Names without a rule raise; LoRA factors are skipped unless `lora_to_hf_mappings` covers them."""
  if config.preprocess_src_state is not None:
    state = config.preprocess_src_state(state)
  out: Dict[str, torch.Tensor] = {}
  rules = list((config.to_hf_mappings or {}).items())
  lora_rules = list((config.lora_to_hf_mappings or {}).items())
  for name, t in state.items():
    is_lora = ".lora_a." in name or ".lora_b." in name
    hit = None
    for pat, (dst, spec) in (lora_rules if is_lora else rules):
      g = _match(pat, name)
      if g is not None:
        hit = (g, dst, spec)
        break
    if hit is None:
      if is_lora:
        continue
      raise KeyError(f"no mapping rule for parameter {name}")
    g, dst, spec = hit
    hook = (config.to_hf_hook_fns or {}).get(name)
    if hook is not None:
      t = hook(t)
    axes = (config.to_hf_transpose_keys or {}).get(name)
    if axes is not None:
      t = t.permute(*axes)
    if spec is not None and spec[0] == "experts":
      inner = spec[1]
      for e in range(t.shape[0]):
        if inner is None:
          out[_fill(dst, list(g) + [e])] = t[e]
        else:
          dim, sections = inner
          pieces = torch.chunk(t[e], sections, dim - 1) if isinstance(sections, int) else \
              torch.split(t[e], list(sections), dim - 1)
          for d, piece in zip(dst, pieces):
            out[_fill(d, list(g) + [e])] = piece
    elif spec is None:
      out[_fill(dst, g)] = t
    else:
      dim, sections = spec
      pieces = torch.chunk(t, sections, dim) if isinstance(sections, int) else torch.split(t, list(sections), dim)
      for d, piece in zip(dst, pieces):
        out[_fill(d, g)] = piece
  return out
