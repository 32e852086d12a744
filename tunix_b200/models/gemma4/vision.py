"""Gemma 4 vision tower (tunix/models/gemma4/vision.py:75-848).

Images arrive as *patches with coordinates*, not as a fixed grid: `patches [B, L, 3 p^2]` (pixel values in 0..1)
and `positions_xy [B, L, 2]` (patch column and row; -1, -1 marks padding), so images of different aspect ratios
share a batch. The tower is

  entry    patches -> 2 (x - 0.5) -> linear to D, plus a factorised position embedding E_x[col] + E_y[row];
  blocks   pre/post-normed attention and gated-GELU MLP (four RMS norms per block); attention has per-head RMS
           norm on q and k (learned scale), a scale-free RMS norm on v, no 1/sqrt(H) factor, and 2-D rotary
           embedding: the first half of every head rotates with the column, the second half with the row
           (base 100); padding patches are masked out as keys;
  exit     average pooling of k x k neighbourhoods *by coordinates* (patch (c, r) goes to cell (c // k, r // k))
           down to `output_length` soft tokens, times sqrt(D); optionally a learned standardisation.

Weights are kept GEMM-ready: q | k | v of all heads as one [3 N H, D] matrix, gate | up as one [2 F, D] matrix, so
a block is four library GEMMs plus `F.attention`. Optional activation clamps around every linear
(`use_clipped_linears`) are buffers loaded from the checkpoint (infinite, i.e. off, by default).
"""
from __future__ import annotations

import dataclasses
import math
from typing import List, Optional, Sequence, Tuple, Union

import torch
from torch import nn

from ...ops import functional as F

POSITIONS_PAD_VALUE = -1
_NORM_EPS = 1e-6
_ROPE_BASE = 100.0


@dataclasses.dataclass
class VisionEncoderConfig:
  d_model: int = 768
  num_layers: int = 16
  num_heads: int = 12
  ffw_hidden: int = 3072
  patch_size: int = 16
  output_length: Union[int, Tuple[int, ...]] = 1120
  pos_emb_shape_yx: Tuple[int, int] = (10240, 2)
  pooling_kernel_size: int = 3
  use_clipped_linears: bool = False
  standardize_embeddings: bool = False

  @property
  def num_mm_tokens_per_image(self) -> int:
    return int(max(self.output_length) if isinstance(self.output_length, tuple) else self.output_length)

  @property
  def max_patches(self) -> int:
    return self.num_mm_tokens_per_image * self.pooling_kernel_size ** 2

  @property
  def image_height(self) -> int:
    return int(self.max_patches ** 0.5) * self.patch_size

  image_width = image_height


# ------------------------------------------------------------------------------------------ functional pieces
def _rms(x: torch.Tensor, scale: Optional[torch.Tensor]) -> torch.Tensor:
  xf = x.float()
  y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + _NORM_EPS)
  return (y * scale.float() if scale is not None else y).to(x.dtype)


def rope_2d(x: torch.Tensor, positions_xy: torch.Tensor, base: float = _ROPE_BASE) -> torch.Tensor:
  """Rotary embedding of [B, L, N, H] heads over two coordinates: channels [0, H/2) rotate with
  `positions_xy[..., 0]`, channels [H/2, H) with `positions_xy[..., 1]`, each as a half-split rotation with
  frequencies base^(-2 i / (H/2))."""
  H = x.shape[-1]
  per = 2 * (H // 4)                                    # rotated channels per coordinate (even)
  parts = []
  for axis in range(2):
    chunk = x[..., axis * per:(axis + 1) * per].float()
    half = per // 2
    inv = base ** (-(2.0 / per) * torch.arange(half, device=x.device, dtype=torch.float32))
    angle = positions_xy[..., axis].float()[..., None, None] * inv          # [B, L, 1, half]
    sin, cos = angle.sin(), angle.cos()
    a, b = chunk[..., :half], chunk[..., half:]
    parts.append(torch.cat((a * cos - b * sin, b * cos + a * sin), dim=-1))
  if 2 * per < H:
    parts.append(x[..., 2 * per:].float())
  return torch.cat(parts, dim=-1).to(x.dtype)


def factorized_posemb(table: torch.Tensor, positions_xy: torch.Tensor) -> torch.Tensor:
  """table [S, 2, D], positions [B, L, 2] -> [B, L, D] = table[col, 0] + table[row, 1]; padding (-1) adds nothing.
  A coordinate beyond the table poisons the row with NaN instead of silently wrapping."""
  S = table.shape[0]
  out = torch.zeros(*positions_xy.shape[:2], table.shape[-1], dtype=table.dtype, device=table.device)
  for axis in range(2):
    idx = positions_xy[..., axis]
    valid = (idx >= 0) & (idx < S)
    gathered = table[idx.clamp(0, S - 1), axis]
    out = out + torch.where(valid[..., None], gathered, torch.zeros_like(gathered))
    beyond = (idx >= S) | (idx < POSITIONS_PAD_VALUE)
    out = torch.where(beyond[..., None], torch.full_like(out, float("nan")), out)
  return out


def avg_pool_by_positions(x: torch.Tensor, positions_xy: torch.Tensor, length: int) -> Tuple[torch.Tensor, torch.Tensor]:
  """[B, L, D] -> ([B, length, D], mask [B, length]): patch (c, r) is averaged into cell
  (c // k) + (r // k) * (columns // k) with k = sqrt(L / length); every cell divides by k^2 (border cells of an
  image whose sides are not multiples of k are therefore damped, as in the reference); cells that received
  nothing are masked."""
  B, L, D = x.shape
  k = int(round((L // length) ** 0.5))
  if k * k * length != L:
    raise ValueError(f"cannot pool {L} patches to {length} tokens")
  cols = positions_xy[..., 0].max(dim=-1, keepdim=True).values + 1
  cell = positions_xy[..., 0] // k + (cols // k) * (positions_xy[..., 1] // k)          # [B, L]
  valid = (positions_xy != POSITIONS_PAD_VALUE).any(dim=-1) & (cell >= 0) & (cell < length)
  target = torch.where(valid, cell, torch.zeros_like(cell))
  weight = valid.to(torch.float32) / (k * k)
  out = torch.zeros(B, length, D, dtype=torch.float32, device=x.device)
  out.scatter_add_(1, target[..., None].expand(B, L, D), x.float() * weight[..., None])
  hits = torch.zeros(B, length, dtype=torch.float32, device=x.device).scatter_add_(1, target, weight)
  return out.to(x.dtype), hits > 0


# ------------------------------------------------------------------------------------------ modules
class ClippedLinear(nn.Module):
  """A linear map whose output rows are grouped in *segments* (q | k | v, gate | up, or a single one), each with
  its own clamps on the input it reads and the output it writes: y_s = clamp(W_s clamp(x)). The bounds are
  checkpoint values (+-inf = no clamp). A model without clamps runs one GEMM over the fused weight; a model with
  clamps runs one GEMM per segment, since segments may clamp the input differently."""

  def __init__(self, out_segments, in_features: int, clipped: bool, dtype, device=None):
    super().__init__()
    self.segments = tuple(out_segments) if isinstance(out_segments, (tuple, list)) else (int(out_segments),)
    self.w = nn.Parameter(torch.zeros(sum(self.segments), in_features, dtype=dtype, device=device))
    self.clipped = clipped
    if clipped:
      S = len(self.segments)
      for name, value in (("clip_input_min", -math.inf), ("clip_input_max", math.inf),
                          ("clip_output_min", -math.inf), ("clip_output_max", math.inf)):
        self.register_buffer(name, torch.full((S,), value, dtype=torch.float32, device=device))

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    if not self.clipped:
      return F.linear(x, self.w)
    outs, row = [], 0
    for s, n in enumerate(self.segments):
      xs = torch.clamp(x, self.clip_input_min[s].to(x.dtype), self.clip_input_max[s].to(x.dtype))
      ys = F.linear(xs, self.w[row:row + n])
      outs.append(torch.clamp(ys, self.clip_output_min[s].to(ys.dtype), self.clip_output_max[s].to(ys.dtype)))
      row += n
    return outs[0] if len(outs) == 1 else torch.cat(outs, dim=-1)


class VisionAttention(nn.Module):

  def __init__(self, cfg: VisionEncoderConfig, dtype, device=None):
    super().__init__()
    self.N, self.H = cfg.num_heads, cfg.d_model // cfg.num_heads
    D = cfg.d_model
    self.qkv_proj = ClippedLinear((self.N * self.H,) * 3, D, cfg.use_clipped_linears, dtype, device)
    self.o_proj = ClippedLinear(D, self.N * self.H, cfg.use_clipped_linears, dtype, device)
    self.query_norm = nn.Parameter(torch.ones(self.H, dtype=dtype, device=device))
    self.key_norm = nn.Parameter(torch.ones(self.H, dtype=dtype, device=device))

  def forward(self, x: torch.Tensor, positions_xy: torch.Tensor, key_mask: torch.Tensor) -> torch.Tensor:
    B, L, _ = x.shape
    q, k, v = self.qkv_proj(x).view(B, L, 3, self.N, self.H).unbind(dim=2)
    q = rope_2d(_rms(q, self.query_norm), positions_xy)
    k = rope_2d(_rms(k, self.key_norm), positions_xy)
    v = _rms(v, None)
    mask = (key_mask[:, :, None] & key_mask[:, None, :])                   # [B, L, L]; padded queries see nothing
    mask = mask | ~key_mask[:, :, None]                                     # ...so let them see everything: no NaN rows
    o = F.attention(q, k, v, mask=mask, causal=False, scale=1.0)
    return self.o_proj(o.reshape(B, L, self.N * self.H))


class VisionMLP(nn.Module):

  def __init__(self, cfg: VisionEncoderConfig, dtype, device=None):
    super().__init__()
    self.gate_up_proj = ClippedLinear((cfg.ffw_hidden,) * 2, cfg.d_model, cfg.use_clipped_linears, dtype, device)
    self.down_proj = ClippedLinear(cfg.d_model, cfg.ffw_hidden, cfg.use_clipped_linears, dtype, device)

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    gate, up = self.gate_up_proj(x).chunk(2, dim=-1)
    return self.down_proj(torch.nn.functional.gelu(gate, approximate="tanh") * up)


class VisionBlock(nn.Module):

  def __init__(self, cfg: VisionEncoderConfig, dtype, device=None):
    super().__init__()
    mk = lambda: nn.Parameter(torch.ones(cfg.d_model, dtype=dtype, device=device))
    self.pre_attention_norm, self.post_attention_norm = mk(), mk()
    self.pre_ffw_norm, self.post_ffw_norm = mk(), mk()
    self.attn = VisionAttention(cfg, dtype, device)
    self.mlp = VisionMLP(cfg, dtype, device)

  def forward(self, x, positions_xy, key_mask):
    h = x + _rms(self.attn(_rms(x, self.pre_attention_norm), positions_xy, key_mask), self.post_attention_norm)
    return h + _rms(self.mlp(_rms(h, self.pre_ffw_norm)), self.post_ffw_norm)


class VisionEncoder(nn.Module):
  """`(patches, positions_xy) -> ((soft tokens [B, length, D], mask [B, length]), ...)`, one pair per configured
  output length that does not exceed the number of patches."""

  def __init__(self, config: VisionEncoderConfig, dtype=torch.float32, device=None):
    super().__init__()
    self.config = config
    D, p = config.d_model, config.patch_size
    self.input_projection = nn.Parameter(torch.zeros(D, 3 * p * p, dtype=dtype, device=device))
    self.pos_emb = nn.Parameter(torch.zeros(config.pos_emb_shape_yx[0], config.pos_emb_shape_yx[1], D, dtype=dtype,
                                            device=device))
    self.layers = nn.ModuleList([VisionBlock(config, dtype, device) for _ in range(config.num_layers)])
    if config.standardize_embeddings:
      self.std_scale = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
      self.std_bias = nn.Parameter(torch.zeros(D, dtype=dtype, device=device))

  def init_weights(self, seed: int = 0, scale: float = 0.02) -> "VisionEncoder":
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
      for p in self.parameters():
        if p.dim() >= 2:
          p.copy_((torch.randn(p.shape, generator=g) * scale).to(p.dtype))
    return self

  max_patches = property(lambda self: self.config.max_patches)
  num_mm_tokens_per_image = property(lambda self: self.config.num_mm_tokens_per_image)
  image_height = property(lambda self: self.config.image_height)
  image_width = property(lambda self: self.config.image_width)

  def embed(self, patches: torch.Tensor, positions_xy: torch.Tensor) -> torch.Tensor:
    x = F.linear((2.0 * (patches - 0.5)).to(self.input_projection.dtype), self.input_projection)
    return x + factorized_posemb(self.pos_emb, positions_xy).to(x.dtype)

  def pool(self, x: torch.Tensor, positions_xy: torch.Tensor, length: int) -> Tuple[torch.Tensor, torch.Tensor]:
    if x.shape[1] == length:
      pooled, mask = x, (positions_xy != POSITIONS_PAD_VALUE).any(dim=-1)
    else:
      pooled, mask = avg_pool_by_positions(x, positions_xy, length)
    pooled = pooled * math.sqrt(self.config.d_model)
    if self.config.standardize_embeddings:
      pooled = ((pooled.float() - self.std_bias.float()) * self.std_scale.float()).to(pooled.dtype)
    return pooled, mask

  def forward(self, patches: torch.Tensor, positions_xy: torch.Tensor):
    key_mask = (positions_xy != POSITIONS_PAD_VALUE).any(dim=-1)
    x = self.embed(patches, positions_xy)
    for block in self.layers:
      x = block(x, positions_xy, key_mask)
    lengths = self.config.output_length
    lengths = (lengths,) if isinstance(lengths, int) else tuple(lengths)
    return tuple(self.pool(x, positions_xy, n) for n in lengths if n <= x.shape[1])


# ------------------------------------------------------------------------------------------ model-side glue
@dataclasses.dataclass
class PreprocessedVisionInput:
  """patches [B, images * max_patches, 3 p^2], positions_xy [B, images * max_patches, 2] and, per batch row, the
  number of soft tokens each of its images occupies in the token sequence."""
  patches: torch.Tensor
  positions_xy: torch.Tensor
  soft_token_counts: Sequence[Sequence[int]]


def soft_tokens_per_row(encoder: VisionEncoder, vision_input: PreprocessedVisionInput) -> Optional[torch.Tensor]:
  """Runs the tower over every image and lines the valid soft tokens of each batch row up in image order:
  [B, max tokens per row, D], zero-padded. None when no row has an image."""
  counts = vision_input.soft_token_counts
  if counts and isinstance(counts[0], int):
    counts = (counts,)
  per_row = max((len(c) for c in counts), default=0)
  if per_row == 0:
    return None
  B = vision_input.patches.shape[0]
  L = vision_input.patches.shape[1] // per_row
  emb, mask = encoder(vision_input.patches.reshape(B * per_row, L, -1),
                      vision_input.positions_xy.reshape(B * per_row, L, 2))[0]
  rows: List[torch.Tensor] = []
  for b in range(B):
    mine = counts[b] if b < len(counts) else ()
    pieces = []
    for i, n in enumerate(mine):
      img = b * per_row + i
      keep = mask[img].nonzero(as_tuple=True)[0][:n]
      piece = emb[img][keep]
      if piece.shape[0] < n:                                # fewer valid cells than announced: pad, never shift
        piece = torch.cat((piece, piece.new_zeros(n - piece.shape[0], piece.shape[1])))
      pieces.append(piece)
    rows.append(torch.cat(pieces) if pieces else emb.new_zeros(0, emb.shape[-1]))
  width = max(r.shape[0] for r in rows)
  return torch.stack([torch.cat((r, r.new_zeros(width - r.shape[0], r.shape[1]))) for r in rows])


def merge_soft_tokens(text: torch.Tensor, soft: torch.Tensor, where: torch.Tensor) -> torch.Tensor:
  """Replaces the embeddings of placeholder positions (`where` [B, T]) by a row's soft tokens, in order."""
  out = text.clone()
  order = where.long().cumsum(dim=1) - 1                                   # index of each placeholder within its row
  b_idx, t_idx = where.nonzero(as_tuple=True)
  src = order[b_idx, t_idx].clamp(max=soft.shape[1] - 1)
  out[b_idx, t_idx] = soft[b_idx, src].to(text.dtype)
  return out
