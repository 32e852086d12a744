"""NF4 weight quantisation for QLoRA (the reference delegates to qwix `weight_qtype="nf4"`
with a `tile_size` block: tunix/cli/utils/model.py:31-77).

Each tile of `tile_size` consecutive input-dim weights shares one absmax scale (fp32); every
weight is stored as the 4-bit index of the nearest of the 16 NormalFloat levels, two per byte.
A quantised projection keeps no bf16 copy of its weight: `Linear.weight()` dequantises on use
(the frozen weight needs no gradient), which cuts its memory from 16 to ~4.5 bits per weight.
"""
from __future__ import annotations

from typing import Iterable, Optional

import torch

# quantiles of N(0,1) normalised to [-1, 1] with an exact zero (the NF4 code book)
NF4_LEVELS = torch.tensor([
    -1.0, -0.6961928009986877, -0.5250730514526367, -0.39491748809814453, -0.28444138169288635,
    -0.18477343022823334, -0.09105003625154495, 0.0, 0.07958029955625534, 0.16093020141124725,
    0.24611230194568634, 0.33791524171829224, 0.44070982933044434, 0.5626170039176941, 0.7229568362236023, 1.0])


class NF4Weight:
  """Packed NF4 form of a `[out, in]` weight."""

  def __init__(self, w: torch.Tensor, tile_size: int = 64):
    out_dim, in_dim = w.shape
    if in_dim % tile_size != 0 or tile_size % 2 != 0:
      raise ValueError(f"input dim {in_dim} must be a multiple of the (even) tile size {tile_size}")
    self.shape, self.dtype, self.tile = (out_dim, in_dim), w.dtype, tile_size
    t = w.detach().float().reshape(out_dim, in_dim // tile_size, tile_size)
    scale = t.abs().amax(-1, keepdim=True).clamp_min(1e-12)
    levels = NF4_LEVELS.to(w.device)
    # nearest level by bucketing at the midpoints
    mids = (levels[1:] + levels[:-1]) / 2
    idx = torch.bucketize((t / scale).contiguous(), mids).to(torch.uint8).reshape(out_dim, in_dim)
    self.packed = (idx[:, 0::2] << 4) | idx[:, 1::2]
    self.scale = scale.squeeze(-1).contiguous()

  def dequantize(self) -> torch.Tensor:
    levels = NF4_LEVELS.to(self.packed.device)
    hi, lo = (self.packed >> 4).long(), (self.packed & 0xF).long()
    idx = torch.stack([hi, lo], -1).reshape(self.shape)
    w = levels[idx].reshape(self.shape[0], -1, self.tile) * self.scale[..., None]
    return w.reshape(self.shape).to(self.dtype)

  def to(self, device) -> "NF4Weight":
    self.packed, self.scale = self.packed.to(device), self.scale.to(device)
    return self

  def nbytes(self) -> int:
    return self.packed.numel() + self.scale.numel() * 4


def quantize_frozen_weights(model: torch.nn.Module, weight_qtype: str = "nf4", tile_size: int = 64,
                            only: Optional[Iterable[torch.nn.Module]] = None) -> torch.nn.Module:
  """Replaces the frozen weight of every adapted projection by its NF4 form."""
  if weight_qtype.lower() != "nf4":
    raise ValueError(f"unsupported weight_qtype {weight_qtype!r}; only 'nf4' is implemented")
  from .transformer import Linear
  mods = list(only) if only is not None else [m for m in model.modules() if isinstance(m, Linear) and len(m.lora_a)]
  seen = set()
  for m in mods:
    if id(m) in seen or m.quant is not None:
      continue
    seen.add(id(m))
    m.quant = NF4Weight(m.w.data, tile_size)
    # the parameter stays registered (names, checkpoints, sharing checks) but holds no storage
    m.w.data = torch.empty(0, dtype=m.w.dtype, device=m.w.device)
    m.w.requires_grad_(False)
  return model
