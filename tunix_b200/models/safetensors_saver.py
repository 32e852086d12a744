"""Saving a (LoRA-merged) model as Hugging Face safetensors.

Role of tunix/models/safetensors_saver.py:29-126: every adapter is folded into its base weight
(W += B·A·alpha/rank), the fused projections are split back into the per-projection HF
tensors, and `config.json` / tokenizer files of the base model directory are copied next to
the weights so that the output directory loads with `from_pretrained`.
"""
from __future__ import annotations

import copy
import os
import shutil
from typing import Dict, Optional

import torch

from . import lora as lora_lib, safetensors_io


def to_hf_state(model: torch.nn.Module) -> Dict[str, torch.Tensor]:
  cfg = model.config
  gemma = cfg.family.startswith("gemma")
  N, K, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
  out: Dict[str, torch.Tensor] = {}
  for name, p in model.named_parameters():
    if getattr(p, "is_lora", False):
      continue
    t = p.detach()
    parts = name.split(".")
    if name == "embedder.input_embedding":
      out["model.embed_tokens.weight"] = t
    elif name == "final_norm.w":
      out["model.norm.weight"] = t
    elif name == "lm_head.w":
      out["lm_head.weight"] = t
    elif parts[0] == "layers":
      pre = f"model.layers.{parts[1]}."
      rest = ".".join(parts[2:])
      if rest in ("attn.qkv_proj.w", "attn.qkv_proj.b"):
        suffix = "weight" if rest.endswith(".w") else "bias"
        q, k, v = torch.split(t, [N * H, K * H, K * H], 0)
        for nm, x in (("q", q), ("k", k), ("v", v)):
          out[f"{pre}self_attn.{nm}_proj.{suffix}"] = x
      elif rest == "attn.o_proj.w":
        out[pre + "self_attn.o_proj.weight"] = t
      elif rest in ("attn.q_norm.w", "attn.k_norm.w"):
        out[f"{pre}self_attn.{parts[3]}.weight"] = t
      elif rest == "input_layernorm.w":
        out[pre + "input_layernorm.weight"] = t
      elif rest == "post_attention_layernorm.w":
        out[pre + ("pre_feedforward_layernorm.weight" if gemma and cfg.use_post_attn_norm else
                   "post_attention_layernorm.weight")] = t
      elif rest == "post_attn_norm.w":
        out[pre + "post_attention_layernorm.weight"] = t
      elif rest == "post_ffw_norm.w":
        out[pre + "post_feedforward_layernorm.weight"] = t
      elif rest == "mlp.gate_up_proj.w":
        g, u = torch.chunk(t, 2, 0)
        out[pre + "mlp.gate_proj.weight"], out[pre + "mlp.up_proj.weight"] = g, u
      elif rest == "mlp.down_proj.w":
        out[pre + "mlp.down_proj.weight"] = t
      elif rest == "mlp.router.w":
        out[pre + "mlp.gate.weight"] = t
      elif rest == "mlp.gate_up_proj":
        for e in range(t.shape[0]):
          g, u = torch.chunk(t[e], 2, 0)
          out[f"{pre}mlp.experts.{e}.gate_proj.weight"] = g
          out[f"{pre}mlp.experts.{e}.up_proj.weight"] = u
      elif rest == "mlp.down_proj":
        for e in range(t.shape[0]):
          out[f"{pre}mlp.experts.{e}.down_proj.weight"] = t[e]
      else:
        raise ValueError(f"no Hugging Face name for parameter {name}")
    else:
      raise ValueError(f"no Hugging Face name for parameter {name}")
  return {k: v.contiguous() for k, v in out.items()}


def save_lora_merged_model_as_safetensors(local_model_path: Optional[str], output_dir: str, lora_model: torch.nn.Module,
                                          rank: Optional[int] = None, alpha: Optional[float] = None,
                                          dtype: Optional[torch.dtype] = None, **unused) -> str:
  """Writes `output_dir/model.safetensors` with adapters merged; `lora_model` is left untouched."""
  del rank, alpha, unused          # each adapter carries its own scale
  merged = lora_lib.merge_lora(copy.deepcopy(lora_model))
  state = to_hf_state(merged)
  if dtype is not None:
    state = {k: v.to(dtype) for k, v in state.items()}
  os.makedirs(output_dir, exist_ok=True)
  out = os.path.join(output_dir, "model.safetensors")
  safetensors_io.save_file(state, out, metadata={"format": "pt"})
  if local_model_path and os.path.isdir(local_model_path):
    for f in os.listdir(local_model_path):
      if f.endswith(".safetensors") or f.endswith(".safetensors.index.json"):
        continue
      src = os.path.join(local_model_path, f)
      if os.path.isfile(src):
        shutil.copy(src, os.path.join(output_dir, f))
  return out
