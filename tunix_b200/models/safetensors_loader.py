"""Hugging Face safetensors -> Transformer weights.

Role of tunix/models/safetensors_loader.py:73-517 and the per-family `params_safetensors.py`:
regex key mapping, fusion of q/k/v and gate/up into the fused projections this decoder uses,
stacking of per-expert MoE weights, dtype cast, tied-embedding handling and a shape check of
every parameter. HF stores Linear weights [out, in], which is this decoder's layout too, so no
transposes are needed; RoPE is half-split in both.
"""
from __future__ import annotations

import re
from typing import Callable, Dict, Iterable, List, Mapping, Optional, Tuple

import torch

from . import safetensors_io

_L = r"model\.layers\.(\d+)\."
_LM = r"(?:language_model\.)?"


def _rules(gemma_norms: bool) -> List[Tuple[re.Pattern, str]]:
  """(pattern over the HF key, staging name). Staging names q/k/v/gate/up are fused afterwards."""
  pre = r"^(?:model\.language_model\.|language_model\.model\.|model\.)"
  lay = pre + r"layers\.(\d+)\."
  rules = [
      (pre + r"embed_tokens\.weight$", "embedder.input_embedding"),
      (pre + r"norm\.weight$", "final_norm.w"),
      (r"^(?:language_model\.)?lm_head\.weight$", "lm_head.w"),
      (lay + r"self_attn\.([qkv])_proj\.weight$", r"layers.\1.attn.\2.w"),
      (lay + r"self_attn\.([qkv])_proj\.bias$", r"layers.\1.attn.\2.b"),
      (lay + r"self_attn\.o_proj\.weight$", r"layers.\1.attn.o_proj.w"),
      (lay + r"self_attn\.([qk])_norm\.weight$", r"layers.\1.attn.\2_norm.w"),
      (lay + r"input_layernorm\.weight$", r"layers.\1.input_layernorm.w"),
      (lay + r"mlp\.(gate|up)_proj\.weight$", r"layers.\1.mlp.\2.w"),
      (lay + r"mlp\.down_proj\.weight$", r"layers.\1.mlp.down_proj.w"),
      (lay + r"mlp\.gate\.weight$", r"layers.\1.mlp.router.w"),
      (lay + r"mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight$", r"layers.\1.mlp.experts.\2.\3"),
      # experts already stacked ([E, 2F, D] gate-then-up and [E, D, F]), as newer exports store them
      (lay + r"mlp\.experts\.gate_up_proj$", r"layers.\1.mlp.gate_up_proj"),
      (lay + r"mlp\.experts\.down_proj$", r"layers.\1.mlp.down_proj"),
  ]
  if gemma_norms:
    rules += [(lay + r"post_attention_layernorm\.weight$", r"layers.\1.post_attn_norm.w"),
              (lay + r"pre_feedforward_layernorm\.weight$", r"layers.\1.post_attention_layernorm.w"),
              (lay + r"post_feedforward_layernorm\.weight$", r"layers.\1.post_ffw_norm.w")]
  else:
    rules += [(lay + r"post_attention_layernorm\.weight$", r"layers.\1.post_attention_layernorm.w")]
  return [(re.compile(p), r) for p, r in rules]


def map_key(key: str, rules) -> Optional[str]:
  for pat, rep in rules:
    if pat.match(key):
      return pat.sub(rep, key)
  return None


def _fuse(staged: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
  out: Dict[str, torch.Tensor] = {}
  groups: Dict[str, Dict[str, torch.Tensor]] = {}
  for name, t in staged.items():
    m = re.match(r"^(layers\.\d+\.attn)\.([qkv])\.(w|b)$", name)
    if m:
      groups.setdefault(f"{m.group(1)}.qkv_proj.{m.group(3)}", {})[m.group(2)] = t
      continue
    m = re.match(r"^(layers\.\d+\.mlp)\.(gate|up)\.w$", name)
    if m:
      groups.setdefault(f"{m.group(1)}.gate_up_proj.w", {})[m.group(2)] = t
      continue
    m = re.match(r"^(layers\.\d+\.mlp)\.experts\.(\d+)\.(gate|up|down)$", name)
    if m:
      groups.setdefault(f"{m.group(1)}.__experts__", {})[f"{m.group(3)}.{int(m.group(2))}"] = t
      continue
    out[name] = t
  for name, parts in groups.items():
    if name.endswith("__experts__"):
      base = name[:-len(".__experts__")]
      n = 1 + max(int(k.split(".")[1]) for k in parts)
      gate_up = [torch.cat([parts[f"gate.{e}"], parts[f"up.{e}"]], 0) for e in range(n)]
      out[f"{base}.gate_up_proj"] = torch.stack(gate_up)                       # [E, 2F, D]
      out[f"{base}.down_proj"] = torch.stack([parts[f"down.{e}"] for e in range(n)])   # [E, D, F]
    elif "qkv_proj" in name:
      out[name] = torch.cat([parts["q"], parts["k"], parts["v"]], 0)
    else:
      out[name] = torch.cat([parts["gate"], parts["up"]], 0)
  return out


def convert_state(tensors: Iterable[Tuple[str, torch.Tensor]], gemma_norms: bool = False,
                  extra_rules: Optional[List[Tuple[str, str]]] = None) -> Tuple[Dict[str, torch.Tensor], List[str]]:
  """-> ({parameter name of `Transformer`: tensor}, [HF keys that no rule matched])."""
  rules = _rules(gemma_norms) + [(re.compile(p), r) for p, r in (extra_rules or [])]
  staged, unmatched = {}, []
  for key, t in tensors:
    name = map_key(key, rules)
    if name is None:
      unmatched.append(key)
    else:
      staged[name] = t
  return _fuse(staged), unmatched


def load_into_model(model: torch.nn.Module, path: str, dtype: Optional[torch.dtype] = None, strict: bool = True,
                    extra_rules: Optional[List[Tuple[str, str]]] = None) -> List[str]:
  """Fills `model` in place from a safetensors file or directory. Returns the ignored HF keys."""
  fam = getattr(getattr(model, "config", None), "family", "")
  state, unmatched = convert_state(safetensors_io.iter_tensors(path), gemma_norms=fam.startswith("gemma"),
                                   extra_rules=extra_rules)
  params = dict(model.named_parameters())
  tied = getattr(model.config, "weight_tying", False)
  missing = [n for n in params if n not in state and not getattr(params[n], "is_lora", False)
             and not (tied and n == "lm_head.w")]
  if strict and missing:
    raise ValueError(f"checkpoint at {path} lacks parameters: {missing[:8]}{'...' if len(missing) > 8 else ''}")
  with torch.no_grad():
    for name, t in state.items():
      if name not in params:
        if name == "lm_head.w" and tied:
          continue
        if strict:
          raise ValueError(f"checkpoint tensor maps to unknown parameter {name}")
        continue
      p = params[name]
      if tuple(t.shape) != tuple(p.shape):
        raise ValueError(f"shape mismatch for {name}: checkpoint {tuple(t.shape)} vs model {tuple(p.shape)}")
      p.copy_(t.to(dtype=dtype or p.dtype))
  return unmatched


def load_and_create_model(file_dir: str, model_class: Callable, config, mesh=None, dtype: Optional[torch.dtype] = None,
                          device: Optional[str] = None, **kw):
  """Builds `model_class(config)` on `device` and loads it (tunix/models/safetensors_loader.py:451-517)."""
  model = model_class(config)
  if dtype is not None:
    model = model.to(dtype)
  if device is not None:
    model = model.to(device)
  load_into_model(model, file_dir, dtype=dtype, **kw)
  return model
