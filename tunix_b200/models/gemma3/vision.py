"""SigLIP vision tower and multimodal wrapper for Gemma 3.

`SigLiP` (tunix/models/gemma3/vision.py:80-682): a ViT - patch embedding by a strided
convolution, learned position embeddings, `depth` pre-LayerNorm blocks (MHA + GELU MLP), final
LayerNorm - whose 4096 patch tokens per 896x896 image are average-pooled 4x4 to 256 soft tokens
(`VisionExit`). `Gemma3Multimodal` projects them to the text width (RMSNorm + linear), writes
them over the placeholder positions of the prompt (tunix/models/gemma3/merge_embeddings.py),
and lets the soft tokens of one image attend to each other in both directions.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as tF


@dataclasses.dataclass
class SigLIPConfig:
  num_mm_tokens_per_image_prepool: int = 4096
  num_mm_tokens_per_image: int = 256
  image_height: int = 896
  image_width: int = 896
  image_channels: int = 3
  image_mean: Tuple[float, ...] = (127.5, 127.5, 127.5)
  image_std: Tuple[float, ...] = (127.5, 127.5, 127.5)
  soft_token_placeholder: int = 219
  patch_size: Tuple[int, int] = (14, 14)
  width: int = 1152
  depth: int = 27
  mlp_dim: Optional[int] = 4304
  num_heads: int = 16
  dropout: float = 0.0


class VisionAttention(nn.Module):

  def __init__(self, width: int, num_heads: int, dtype=None, device=None):
    super().__init__()
    if width % num_heads:
      raise ValueError(f"width {width} is not divisible by {num_heads} heads")
    self.num_heads = num_heads
    self.qkv = nn.Linear(width, 3 * width, dtype=dtype, device=device)
    self.out = nn.Linear(width, width, dtype=dtype, device=device)

  def forward(self, x):
    B, L, D = x.shape
    q, k, v = self.qkv(x).view(B, L, 3, self.num_heads, D // self.num_heads).unbind(2)
    o = tF.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    return self.out(o.transpose(1, 2).reshape(B, L, D))


class Encoder1DBlock(nn.Module):

  def __init__(self, width: int, mlp_dim: int, num_heads: int, dropout: float, dtype=None, device=None):
    super().__init__()
    self.ln1 = nn.LayerNorm(width, eps=1e-6, dtype=dtype, device=device)
    self.attn = VisionAttention(width, num_heads, dtype, device)
    self.ln2 = nn.LayerNorm(width, eps=1e-6, dtype=dtype, device=device)
    self.fc1 = nn.Linear(width, mlp_dim, dtype=dtype, device=device)
    self.fc2 = nn.Linear(mlp_dim, width, dtype=dtype, device=device)
    self.drop = nn.Dropout(dropout)

  def forward(self, x):
    x = x + self.drop(self.attn(self.ln1(x)))
    y = self.fc2(self.drop(tF.gelu(self.fc1(self.ln2(x)), approximate="tanh")))
    return x + self.drop(y)


class ViTModel(nn.Module):

  def __init__(self, cfg: SigLIPConfig, dtype=None, device=None):
    super().__init__()
    ph, pw = cfg.patch_size
    self.embedding = nn.Conv2d(cfg.image_channels, cfg.width, (ph, pw), stride=(ph, pw), dtype=dtype, device=device)
    n = (cfg.image_height // ph) * (cfg.image_width // pw)
    self.pos_embedding = nn.Parameter(torch.zeros(1, n, cfg.width, dtype=dtype, device=device))
    mlp = cfg.mlp_dim or 4 * cfg.width
    self.blocks = nn.ModuleList(Encoder1DBlock(cfg.width, mlp, cfg.num_heads, cfg.dropout, dtype, device)
                                for _ in range(cfg.depth))
    self.encoder_norm = nn.LayerNorm(cfg.width, eps=1e-6, dtype=dtype, device=device)

  def forward(self, image):            # [B, H, W, C] channel-last, as the processor produces it
    x = self.embedding(image.permute(0, 3, 1, 2).to(self.pos_embedding.dtype))
    x = x.flatten(2).transpose(1, 2) + self.pos_embedding
    for blk in self.blocks:
      x = blk(x)
    return self.encoder_norm(x)


class VisionExit(nn.Module):
  """Spatial average pooling of the patch grid down to `output_length` tokens."""

  def __init__(self, output_length: int = 256):
    super().__init__()
    self.output_length = output_length

  def forward(self, x):
    B, L, D = x.shape
    if L == self.output_length:
      return x
    side, out_side = int(math.isqrt(L)), int(math.isqrt(self.output_length))
    win = side // out_side
    x = x.view(B, side, side, D).permute(0, 3, 1, 2)
    x = tF.avg_pool2d(x, win, win)
    return x.permute(0, 2, 3, 1).reshape(B, out_side * out_side, D)


class SigLiP(nn.Module):

  def __init__(self, config: SigLIPConfig, apply_stop_gradient: bool = True, dtype=None, device=None):
    super().__init__()
    self.config = config
    self.apply_stop_gradient = apply_stop_gradient
    self.siglip_encoder = ViTModel(config, dtype, device)
    self.siglip_exit = VisionExit(config.num_mm_tokens_per_image)

  def forward(self, images):           # [B, N, H, W, C] -> [B, N, tokens, width]
    B, N = images.shape[:2]
    tok = self.siglip_encoder(images.reshape(B * N, *images.shape[2:]))
    if tok.shape[1] != self.config.num_mm_tokens_per_image:
      tok = self.siglip_exit(tok)
    tok = tok.view(B, N, *tok.shape[1:])
    return tok.detach() if self.apply_stop_gradient else tok


def merge_embeddings(text_embeddings: torch.Tensor, vision_embeddings: torch.Tensor, mask: torch.Tensor):
  """Writes the soft tokens (in image order) over the positions where `mask` [B, L] is true.
  A row uses as many soft tokens as it has placeholders; text [B, L, D], vision [B, N, P, D]."""
  B, L, D = text_embeddings.shape
  flat = vision_embeddings.reshape(B, -1, D).to(text_embeddings.dtype)
  rank = torch.cumsum(mask.long(), dim=1) - 1                     # index of each placeholder within its row
  rank = rank.clamp(0, flat.shape[1] - 1)
  picked = torch.gather(flat, 1, rank[..., None].expand(B, L, D))
  return torch.where(mask[..., None], picked, text_embeddings)


def multimodal_attention_mask(tokens: torch.Tensor, placeholder: int, tokens_per_image: int,
                              pad_id: Optional[int] = None) -> torch.Tensor:
  """[B, L, L] bool: causal, plus both directions between the soft tokens of the same image (runs of
  `tokens_per_image` consecutive placeholders)."""
  B, L = tokens.shape
  causal = torch.ones(L, L, dtype=torch.bool, device=tokens.device).tril()[None].expand(B, L, L)
  is_img = tokens == placeholder
  img_id = (torch.cumsum(is_img.long(), dim=1) - 1) // max(tokens_per_image, 1)
  same = is_img[:, :, None] & is_img[:, None, :] & (img_id[:, :, None] == img_id[:, None, :])
  mask = causal | same
  if pad_id is not None:
    mask = mask & (tokens != pad_id)[:, None, :]
  return mask


class Gemma3Multimodal(nn.Module):
  """Text decoder + SigLIP. `forward(input_tokens, images=...)`: prompts carry
  `vision.config.soft_token_placeholder` where image tokens go (256 per image)."""

  def __init__(self, text_model: nn.Module, vision_config: Optional[SigLIPConfig] = None, dtype=None, device=None):
    super().__init__()
    self.text = text_model
    self.config = text_model.config
    self.vision_config = vision_config or SigLIPConfig()
    dtype = dtype or self.config.dtype
    self.vision_encoder = SigLiP(self.vision_config, dtype=dtype, device=device)
    from ..transformer import RMSNorm
    self.mm_soft_embedding_norm = RMSNorm(self.vision_config.width, self.config.norm_eps, self.config.norm_offset,
                                          dtype, device)
    self.mm_input_projection = nn.Parameter(
        torch.zeros(self.config.embed_dim, self.vision_config.width, dtype=dtype, device=device))

  def encode_images(self, images: torch.Tensor) -> torch.Tensor:
    soft = self.vision_encoder(images)
    soft = self.mm_soft_embedding_norm(soft)
    return tF.linear(soft, self.mm_input_projection)

  def forward(self, input_tokens, positions=None, cache=None, attention_mask=None, images=None, **kw):
    if images is None:
      return self.text(input_tokens, positions, cache, attention_mask, **kw)
    ph = self.vision_config.soft_token_placeholder
    is_img = input_tokens == ph
    text = self.text.embedder.encode(torch.where(is_img, torch.zeros_like(input_tokens), input_tokens))
    merged = merge_embeddings(text, self.encode_images(images), is_img)
    if attention_mask is None and cache is None:
      attention_mask = multimodal_attention_mask(input_tokens, ph, self.vision_config.num_mm_tokens_per_image)
    return self.text(input_tokens, positions, cache, attention_mask, input_embeddings=merged, **kw)


# ---------------------------------------------------------------------------------------------------------
# Hugging Face checkpoint import (Gemma3ForConditionalGeneration: SigLIP tower + projector + text decoder)
_VISION_PREFIXES = ("model.vision_tower.vision_model.", "vision_tower.vision_model.")
_PROJ_PREFIXES = ("model.multi_modal_projector.", "multi_modal_projector.")
_TEXT_PREFIXES = ("model.language_model.", "language_model.model.")


def _strip(key: str, prefixes) -> Optional[str]:
  for p in prefixes:
    if key.startswith(p):
      return key[len(p):]
  return None


def convert_hf_multimodal_state(tensors) -> Tuple[dict, dict, list]:
  """Splits a Hugging Face multimodal state dict into (vision + projector tensors under this module's
  parameter names, text tensors under the names of a text-only Gemma 3 checkpoint, unused keys).

  q/k/v projections of a SigLIP layer are fused row-wise into `attn.qkv`; the projector matrix is stored by
  HF as [vision width, text width] and used as `x @ W`, here as a [text, vision] `linear` weight; the
  attention-pooling head of the SigLIP checkpoint is not part of Gemma 3 and is reported as unused."""
  import re
  vis, text, unused, qkv = {}, {}, [], {}
  for key, t in tensors:
    v = _strip(key, _VISION_PREFIXES)
    if v is not None:
      if v.startswith("head."):
        unused.append(key)
      elif v == "embeddings.patch_embedding.weight":
        vis["vision_encoder.siglip_encoder.embedding.weight"] = t
      elif v == "embeddings.patch_embedding.bias":
        vis["vision_encoder.siglip_encoder.embedding.bias"] = t
      elif v == "embeddings.position_embedding.weight":
        vis["vision_encoder.siglip_encoder.pos_embedding"] = t[None]
      elif v.startswith("post_layernorm."):
        vis["vision_encoder.siglip_encoder.encoder_norm." + v.split(".", 1)[1]] = t
      else:
        m = re.match(r"encoder\.layers\.(\d+)\.(.+)\.(weight|bias)$", v)
        if not m:
          unused.append(key)
          continue
        i, name, kind = m.group(1), m.group(2), m.group(3)
        base = f"vision_encoder.siglip_encoder.blocks.{i}."
        simple = {"layer_norm1": "ln1", "layer_norm2": "ln2", "mlp.fc1": "fc1", "mlp.fc2": "fc2",
                  "self_attn.out_proj": "attn.out"}
        if name in simple:
          vis[base + simple[name] + "." + kind] = t
        elif name in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"):
          qkv.setdefault((i, kind), {})[name[-6]] = t
        else:
          unused.append(key)
      continue
    pj = _strip(key, _PROJ_PREFIXES)
    if pj is not None:
      if pj == "mm_input_projection_weight":
        vis["mm_input_projection"] = t.t().contiguous()
      elif pj == "mm_soft_emb_norm.weight":
        vis["mm_soft_embedding_norm.w"] = t
      else:
        unused.append(key)
      continue
    tx = _strip(key, _TEXT_PREFIXES)
    if tx is not None:
      text["model." + tx] = t
    else:
      text[key] = t                     # lm_head.weight and text-only checkpoints pass through
  for (i, kind), parts in qkv.items():
    vis[f"vision_encoder.siglip_encoder.blocks.{i}.attn.qkv.{kind}"] = torch.cat([parts["q"], parts["k"], parts["v"]], 0)
  return vis, text, unused


def load_hf_multimodal_state(model: "Gemma3Multimodal", tensors) -> list:
  """Copies a Hugging Face `Gemma3ForConditionalGeneration` state dict into `model`; returns the unused keys."""
  from .. import safetensors_loader
  vis, text, unused = convert_hf_multimodal_state(tensors)
  tstate, unmatched = safetensors_loader.convert_state(text.items(), gemma_norms=True)
  own = dict(model.named_parameters())
  with torch.no_grad():
    for n, t in vis.items():
      if n not in own:
        raise KeyError(f"checkpoint tensor maps to {n!r}, which this model does not have")
      if tuple(own[n].shape) != tuple(t.shape):
        raise ValueError(f"{n}: checkpoint {tuple(t.shape)} vs model {tuple(own[n].shape)}")
      own[n].copy_(t)
    for n, p in model.text.named_parameters():
      if n in tstate:
        p.copy_(tstate[n])
      elif not (n == "lm_head.w" and model.config.weight_tying):
        raise KeyError(f"{n} missing from the checkpoint")
  return unused + list(unmatched)
