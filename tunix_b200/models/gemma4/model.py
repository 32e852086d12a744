"""Gemma 4 text decoder (tunix/models/gemma4/{config,model,attention,layers,moe}.py).

What sets the family apart from Gemma 3, and how it is built here:

* layer pattern of N local sliding-window layers followed by one global layer; global layers may use
  their own key size (`global_key_size`, default 512), their own number of KV heads and `k == v`
  (one projection feeds both); partial RoPE: only the first `rope_proportion` of the frequency pairs
  rotate (0.25 on global layers), the rest pass through;
* q and k are RMS-normalised per head (learned scale, initialised to one: plain `w * x / rms`), v is
  RMS-normalised without a scale, and attention uses no 1/sqrt(H) factor;
* KV sharing: the last `frac_shared_layers` of the stack own no K/V - a shared local layer attends to
  the K/V of the last unshared local layer, a shared global layer to those of the last unshared
  global layer (`kv_sharing_pattern`); shared layers may have a wider MLP;
* per-layer inputs: every layer receives a small [P]-vector per token (a slice of a second embedding
  table plus a projection of the first embedding), gated by gelu(W h) and added after the MLP;
* optional MoE branch in parallel with the dense MLP (top-k of a softmax router over an RMS-normalised,
  scaled input; GeGLU experts; a learned per-expert output scale), each branch with its own norms;
* every layer output is multiplied by a learned scalar; final logits are soft-capped at 30.

The module is plain PyTorch on top of `ops.functional` (the attention core goes through `F.attention`,
so CUDA runs use the same kernels as the other families where the head size allows). Vision and audio
towers are not part of this file. KV cache: `{layer_i: {k, v, end_index}}` for unshared layers only.
"""
from __future__ import annotations

import dataclasses
import enum
import itertools
import math
from typing import Dict, List, Optional, Tuple

import torch
from torch import nn

from ...ops import functional as F


class AttentionType(enum.Enum):
  GLOBAL = 1
  LOCAL_SLIDING = 2


_L, _G = AttentionType.LOCAL_SLIDING, AttentionType.GLOBAL
PATTERN_5_1 = (_L, _L, _L, _L, _L, _G)
PATTERN_4_1 = (_L, _L, _L, _L, _G)


@dataclasses.dataclass
class ModelConfig:
  num_layers: int
  num_embed: int
  embed_dim: int
  hidden_dim: int
  num_heads: int
  head_dim: int
  num_kv_heads: int
  final_logit_softcap: Optional[float] = 30.0
  vision_encoder: Optional[object] = None          # vision.VisionEncoderConfig: adds the image tower
  audio_encoder: Optional[object] = None           # audio.ConformerConfig: adds the audio tower
  use_bidirectional_attention: Optional[str] = None   # "vision": image tokens of one image see each other in local layers
  sliding_window_size: Optional[int] = None
  use_sliding_window_kv_cache: bool = False    # local layers keep only a window-sized ring of keys / values
  per_layer_input_dim: int = 0
  num_global_kv_heads: Optional[int] = None
  global_key_size: Optional[int] = 512
  attention_pattern: Tuple[AttentionType, ...] = PATTERN_5_1
  frac_shared_layers: float = 0.0
  global_rope_proportion: float = 0.25
  local_rope_proportion: float = 1.0
  k_eq_v_global: bool = False
  override_kv_shared_ffw_hidden: Optional[int] = None
  local_base_frequency: float = 10_000.0
  global_base_frequency: float = 1_000_000.0
  local_scale_factor: float = 1.0
  global_scale_factor: float = 1.0
  enable_moe: bool = False
  num_experts: Optional[int] = None
  num_experts_per_tok: Optional[int] = None
  expert_dim: Optional[int] = None
  dtype: torch.dtype = torch.float32
  norm_eps: float = 1e-6

  @property
  def vocab_size(self) -> int:
    return self.num_embed

  def replace(self, **kw) -> "ModelConfig":
    return dataclasses.replace(self, **kw)

  def attention_types(self) -> List[AttentionType]:
    return [t for _, t in zip(range(self.num_layers), itertools.cycle(self.attention_pattern))]

  # ---- presets (tunix/models/gemma4/config.py:188-345) -----------------------------------
  @classmethod
  def gemma4_e2b(cls) -> "ModelConfig":
    return cls(num_layers=35, num_embed=262144, embed_dim=1536, hidden_dim=1536 * 4, num_heads=8, head_dim=256,
               num_kv_heads=1, sliding_window_size=512, per_layer_input_dim=256, frac_shared_layers=20.0 / 35,
               override_kv_shared_ffw_hidden=1536 * 4 * 2, attention_pattern=PATTERN_4_1)

  @classmethod
  def gemma4_e4b(cls) -> "ModelConfig":
    return cls(num_layers=42, num_embed=262144, embed_dim=2560, hidden_dim=2560 * 4, num_heads=8, head_dim=256,
               num_kv_heads=2, sliding_window_size=512, per_layer_input_dim=256, frac_shared_layers=18.0 / 42)

  @classmethod
  def gemma4_12b(cls) -> "ModelConfig":
    return cls(num_layers=48, num_embed=262144, embed_dim=3840, hidden_dim=3840 * 4, num_heads=16, head_dim=256,
               num_kv_heads=8, num_global_kv_heads=1, sliding_window_size=1024, k_eq_v_global=True)

  @classmethod
  def gemma4_31b(cls) -> "ModelConfig":
    return cls(num_layers=60, num_embed=262144, embed_dim=5376, hidden_dim=5376 * 4, num_heads=32, head_dim=256,
               num_kv_heads=16, num_global_kv_heads=4, sliding_window_size=1024, k_eq_v_global=True)

  @classmethod
  def gemma4_26b_a4b(cls) -> "ModelConfig":
    return cls(num_layers=30, num_embed=262144, embed_dim=2816, hidden_dim=2112, num_heads=16, head_dim=256,
               num_kv_heads=8, num_global_kv_heads=2, sliding_window_size=1024, enable_moe=True, num_experts=128,
               expert_dim=704, num_experts_per_tok=8, k_eq_v_global=True)


_PRESETS = ("gemma4_e2b", "gemma4_e4b", "gemma4_12b", "gemma4_31b", "gemma4_26b_a4b")
for _name in _PRESETS:
  setattr(ModelConfig, _name + "_it", getattr(ModelConfig, _name))
ModelConfig.preset_names = classmethod(lambda cls: [n + s for n in _PRESETS for s in ("", "_it")])


def kv_sharing_pattern(num_layers: int, frac_shared_layers: float, types: List[AttentionType]) -> List[int]:
  """For every layer, the index of the layer whose K/V it attends to (itself unless shared): a shared global
  layer uses the last unshared layer, a shared local layer the one before it."""
  unshared = int(num_layers - frac_shared_layers * num_layers)
  out = []
  for i in range(num_layers):
    if i < unshared:
      out.append(i)
    elif types[i] == AttentionType.GLOBAL:
      out.append(unshared - 1)
    else:
      out.append(unshared - 2)
  return out


def _param(*shape, dtype, device=None, ones=False):
  t = torch.ones(*shape, dtype=dtype, device=device) if ones else torch.zeros(*shape, dtype=dtype, device=device)
  return nn.Parameter(t)


def rms(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
  """x / rms(x) in fp32, times `w` when given (no +1 offset in this family)."""
  xf = x.float()
  y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
  if w is not None:
    y = y * w.float()
  return y.to(x.dtype)


def partial_rope(x: torch.Tensor, positions: torch.Tensor, base: float, scale: float, proportion: float):
  """Half-split RoPE on [B, T, N, H] where only the first int(proportion * H / 2) frequency pairs rotate."""
  H = x.shape[-1]
  n_rot = int(proportion * H // 2)
  inv = torch.zeros(H // 2, dtype=torch.float32, device=x.device)
  inv[:n_rot] = base ** (-(2.0 / H) * torch.arange(n_rot, dtype=torch.float32, device=x.device))
  ang = positions[..., None].float() * inv / scale          # [B, T, H/2]; zero angle = identity
  sin, cos = ang.sin()[:, :, None, :], ang.cos()[:, :, None, :]
  a, b = x.float().chunk(2, dim=-1)
  return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)


class Attention(nn.Module):

  def __init__(self, cfg: ModelConfig, attn_type: AttentionType, owns_kv: bool, device=None):
    super().__init__()
    self.cfg, self.attn_type = cfg, attn_type
    glob = attn_type == AttentionType.GLOBAL
    self.rope_proportion = cfg.global_rope_proportion if glob else cfg.local_rope_proportion
    self.rope_base = cfg.global_base_frequency if glob else cfg.local_base_frequency
    self.rope_scale = cfg.global_scale_factor if glob else cfg.local_scale_factor
    self.num_kv_heads = cfg.num_global_kv_heads if (glob and cfg.num_global_kv_heads) else cfg.num_kv_heads
    self.head_dim = cfg.global_key_size if (glob and cfg.global_key_size) else cfg.head_dim
    N, K, H, D = cfg.num_heads, self.num_kv_heads, self.head_dim, cfg.embed_dim
    kw = dict(dtype=cfg.dtype, device=device)
    self.q_proj = _param(N * H, D, **kw)
    self.o_proj = _param(D, N * H, **kw)
    self.k_eq_v = glob and cfg.k_eq_v_global
    if owns_kv:
      self.k_proj = _param(K * H, D, **kw)
      self.v_proj = None if self.k_eq_v else _param(K * H, D, **kw)
      self.k_norm = _param(H, ones=True, **kw)
    else:
      self.k_proj = self.v_proj = self.k_norm = None
    self.q_norm = _param(H, ones=True, **kw)

  def project_kv(self, x, positions):
    cfg = self.cfg
    B, T, _ = x.shape
    K, H = self.num_kv_heads, self.head_dim
    k = F.linear(x, self.k_proj).view(B, T, K, H)
    v = k if self.k_eq_v else F.linear(x, self.v_proj).view(B, T, K, H)
    v = rms(v, None, cfg.norm_eps)
    k = partial_rope(rms(k, self.k_norm, cfg.norm_eps), positions, self.rope_base, self.rope_scale,
                     self.rope_proportion)
    return k, v

  def forward(self, x, positions, cache, attn_mask, shared_kv=None, slot_keys: bool = False):
    """attn_mask: [B, T, S] bool over the keys the layer sees (S = T without a cache, the cache length with one),
    or None for causal attention. `slot_keys`: the keys are cache slots (slot index == absolute position while
    the cache has not wrapped) rather than this call's tokens. Returns (new_cache, out, (k, v))."""
    cfg = self.cfg
    B, T, _ = x.shape
    N, H = cfg.num_heads, self.head_dim
    q = F.linear(x, self.q_proj).view(B, T, N, H)
    q = partial_rope(rms(q, self.q_norm, cfg.norm_eps), positions, self.rope_base, self.rope_scale,
                     self.rope_proportion)
    new_cache = None
    ring = (cfg.use_sliding_window_kv_cache and self.attn_type == AttentionType.LOCAL_SLIDING
            and bool(cfg.sliding_window_size))
    newest = None                      # ring decode: absolute position of the token being decoded, [B]
    if shared_kv is not None:
      k, v = shared_kv["k"], shared_kv["v"]
      if ring and T == 1 and "end_index" in shared_kv:
        newest = shared_kv["end_index"] - 1          # the owner of these keys has already counted this token
    else:
      k, v = self.project_kv(x, positions)
      if cache is not None:
        S = cache["k"].shape[1]
        keep = min(T, S)                             # a prompt longer than the ring leaves its last S tokens
        idx = (cache["end_index"][:, None] + torch.arange(T - keep, T, device=x.device)[None]) % S
        bidx = torch.arange(B, device=x.device)[:, None].expand(B, keep)
        ck = cache["k"].index_put((bidx, idx), k[:, T - keep:].to(cache["k"].dtype))
        cv = cache["v"].index_put((bidx, idx), v[:, T - keep:].to(cache["v"].dtype))
        new_cache = {"k": ck, "v": cv, "end_index": cache["end_index"] + T}
        if ring and T > 1:
          slot_keys = False                          # prefill attends this call's own keys; the ring only records
        else:
          k, v = ck, cv
          if ring:
            newest = cache["end_index"]
    S = k.shape[1]
    mask = attn_mask
    if newest is not None:
      # ring decode: slot p holds absolute position newest - ((newest - p) mod S); slots never written are < 0
      slots = torch.arange(S, device=x.device)[None, :]
      logical = newest[:, None] - ((newest[:, None] - slots) % S)                       # [B, S]
      written = logical >= 0
      seen = written & (logical > newest[:, None] - cfg.sliding_window_size)
      if mask is not None:                           # the caller's mask speaks about absolute positions
        seen = seen & torch.gather(mask[:, 0, :], 1, logical.clamp(min=0, max=mask.shape[-1] - 1))
      mask = seen[:, None, :]
    else:
      slot_keys = slot_keys or (cache is not None and not (ring and T > 1))
      kpos = torch.arange(S, device=x.device)[None, None, :] if slot_keys else positions[:, None, :]
      qpos = positions[:, :, None]
      if slot_keys and mask is None:
        mask = kpos <= qpos                    # written slots up to the query's own position
      if self.attn_type == AttentionType.LOCAL_SLIDING and cfg.sliding_window_size:
        win = (kpos > qpos - cfg.sliding_window_size) & (kpos <= qpos)     # the window behind the query
        mask = win if mask is None else (mask[..., :S] & win)
    causal = mask is None
    o = F.attention(q, k, v, mask=mask, causal=causal, scale=1.0)
    out = F.linear(o.reshape(B, T, N * H), self.o_proj)
    return new_cache, out, (k, v)


class FeedForward(nn.Module):

  def __init__(self, cfg: ModelConfig, hidden: int, device=None):
    super().__init__()
    kw = dict(dtype=cfg.dtype, device=device)
    self.gate_up_proj = _param(2 * hidden, cfg.embed_dim, **kw)      # [gate | up] rows
    self.down_proj = _param(cfg.embed_dim, hidden, **kw)

  def forward(self, x):
    return F.linear(F.glu(F.linear(x, self.gate_up_proj), "gelu"), self.down_proj)


class MoE(nn.Module):
  """Top-k routed GeGLU experts with a per-expert output scale (tunix/models/gemma4/moe.py:80-217)."""

  def __init__(self, cfg: ModelConfig, device=None):
    super().__init__()
    self.cfg = cfg
    E, D, Fe = cfg.num_experts, cfg.embed_dim, cfg.expert_dim
    kw = dict(dtype=cfg.dtype, device=device)
    self.router = _param(E, D, **kw)
    self.router_scale = _param(D, ones=True, **kw)
    self.gate_up_proj = _param(E, 2 * Fe, D, **kw)
    self.down_proj = _param(E, D, Fe, **kw)
    self.per_expert_scale = _param(E, ones=True, **kw)

  def route(self, router_input: torch.Tensor):
    cfg = self.cfg
    r = rms(router_input, None, cfg.norm_eps) * (cfg.embed_dim ** -0.5) * self.router_scale
    logits = F.linear(r, self.router).float()
    probs = torch.softmax(logits, dim=-1)
    _, topi = torch.topk(logits, cfg.num_experts_per_tok, dim=-1)
    picked = probs.gather(-1, topi)
    denom = picked.sum(-1, keepdim=True)
    return picked / torch.where(denom > 0, denom, torch.ones_like(denom)), topi

  def forward(self, x, router_input=None):
    from ...ops import moe as moe_ops
    B, T, D = x.shape
    x2 = x.reshape(B * T, D)
    topv, topi = self.route((x if router_input is None else router_input).reshape(B * T, D))
    topv = topv * self.per_expert_scale.float()[topi]        # the expert's output scale folds into its weight
    if moe_ops.grouped_supported(x2, self.gate_up_proj) and moe_ops.grouped_supported(x2, self.down_proj):
      return moe_ops.moe_forward_padded(x2, topv, topi, self.gate_up_proj, self.down_proj, "gelu").view(B, T, D)
    k = topi.shape[1]
    flat = topi.reshape(-1)
    order = torch.argsort(flat, stable=True)
    tok = order // k
    counts = torch.bincount(flat, minlength=self.cfg.num_experts).tolist()
    ys = moe_ops.grouped_mlp(x2.index_select(0, tok), counts, self.gate_up_proj, self.down_proj, "gelu")
    w = topv.reshape(-1).index_select(0, order).to(ys.dtype)
    return torch.zeros_like(x2).index_add_(0, tok, ys * w[:, None]).view(B, T, D)


class DecoderLayer(nn.Module):

  def __init__(self, cfg: ModelConfig, attn_type: AttentionType, hidden: int, owns_kv: bool, device=None):
    super().__init__()
    self.cfg = cfg
    D = cfg.embed_dim
    norm = lambda: _param(D, ones=True, dtype=cfg.dtype, device=device)
    self.pre_attention_norm, self.post_attention_norm = norm(), norm()
    self.pre_ffw_norm, self.post_ffw_norm = norm(), norm()
    self.attn = Attention(cfg, attn_type, owns_kv, device)
    self.mlp = FeedForward(cfg, hidden, device)
    if cfg.enable_moe:
      self.moe_pre_ffw_norm, self.moe_post_ffw_norm, self.dense_post_ffw_norm = norm(), norm(), norm()
      self.moe = MoE(cfg, device)
    if cfg.per_layer_input_dim > 0:
      P = cfg.per_layer_input_dim
      self.per_layer_input_gate = _param(P, D, dtype=cfg.dtype, device=device)
      self.per_layer_projection = _param(D, P, dtype=cfg.dtype, device=device)
      self.post_per_layer_input_norm = norm()
    self.skip_scale = _param(1, ones=True, dtype=cfg.dtype, device=device)

  def forward(self, x, positions, cache, attn_mask, per_layer_input=None, shared_kv=None, slot_keys: bool = False):
    eps = self.cfg.norm_eps
    new_cache, a, kv = self.attn(rms(x, self.pre_attention_norm, eps), positions, cache, attn_mask, shared_kv,
                                 slot_keys)
    a = rms(a, self.post_attention_norm, eps) + x
    f = self.mlp(rms(a, self.pre_ffw_norm, eps))
    if self.cfg.enable_moe:
      f = rms(f, self.dense_post_ffw_norm, eps)
      m = self.moe(rms(a, self.moe_pre_ffw_norm, eps), router_input=a)
      f = f + rms(m, self.moe_post_ffw_norm, eps)
    f = rms(f, self.post_ffw_norm, eps) + a
    if self.cfg.per_layer_input_dim > 0 and per_layer_input is not None:
      g = torch.nn.functional.gelu(F.linear(f, self.per_layer_input_gate), approximate="tanh") * per_layer_input
      f = f + rms(F.linear(g, self.per_layer_projection), self.post_per_layer_input_norm, eps)
    return new_cache, f * self.skip_scale, kv


IMAGE_SOFT_TOKEN_PLACEHOLDER = -2
AUDIO_SOFT_TOKEN_PLACEHOLDER = -4


def add_bidirectional_blocks(attn_mask: torch.Tensor, member: torch.Tensor) -> torch.Tensor:
  """Opens `attn_mask` [B, T, S] between positions of the same run of consecutive `member` tokens ([B, T]): the
  soft tokens of one image attend to each other in both directions; different images stay causal."""
  starts = member & ~torch.nn.functional.pad(member, (1, 0))[:, :-1]
  block = torch.where(member, starts.long().cumsum(dim=1), torch.zeros_like(starts, dtype=torch.long))    # 0 = not a member
  q = block
  S = attn_mask.shape[-1]
  k = block if S == block.shape[1] else (torch.nn.functional.pad(block, (0, S - block.shape[1]))
                                          if S > block.shape[1] else block[:, -S:])
  same = (q[:, :, None] == k[:, None, :]) & (q[:, :, None] > 0)
  return attn_mask | same


class Embedder(nn.Module):

  def __init__(self, cfg: ModelConfig, device=None):
    super().__init__()
    self.cfg = cfg
    kw = dict(dtype=cfg.dtype, device=device)
    self.input_embedding = _param(cfg.num_embed, cfg.embed_dim, **kw)
    if cfg.per_layer_input_dim > 0:
      LP = cfg.num_layers * cfg.per_layer_input_dim
      self.per_layer_model_projection = _param(LP, cfg.embed_dim, **kw)
      self.per_layer_projection_norm = _param(cfg.per_layer_input_dim, ones=True, **kw)
      self.per_layer_input_embedding = _param(cfg.num_embed, LP, **kw)
    if cfg.vision_encoder is not None:
      self.mm_input_projection = _param(cfg.embed_dim, cfg.vision_encoder.d_model, **kw)
    if cfg.audio_encoder is not None:
      self.audio_input_projection = _param(cfg.embed_dim, cfg.audio_encoder.lm_model_dims, **kw)

  def encode(self, tokens):
    # multimodal placeholders are negative ids: they embed as token 0 and are overwritten by soft tokens
    safe = torch.where(tokens >= 0, tokens, torch.zeros_like(tokens))
    return F.embedding(safe, self.input_embedding, math.sqrt(self.cfg.embed_dim))

  def encode_vision(self, soft):
    """Tower output -> text embedding space: scale-free RMS norm, then a linear map."""
    return F.linear(rms(soft, None, self.cfg.norm_eps).to(self.mm_input_projection.dtype), self.mm_input_projection)

  def encode_audio(self, soft):
    """Audio tower output -> text embedding space: linear map, then a scale-free RMS norm."""
    return rms(F.linear(soft.to(self.audio_input_projection.dtype), self.audio_input_projection), None, self.cfg.norm_eps)

  def encode_per_layer_input(self, x, tokens):
    """[B, T, L, P]: (norm(proj(x) / sqrt(D)) + sqrt(P) * table[token]) / sqrt(2)."""
    cfg = self.cfg
    L, P = cfg.num_layers, cfg.per_layer_input_dim
    t = torch.where((tokens >= 0) & (tokens < cfg.num_embed), tokens, torch.zeros_like(tokens))
    a = F.linear(x, self.per_layer_model_projection) * (cfg.embed_dim ** -0.5)
    a = rms(a.view(*a.shape[:-1], L, P), self.per_layer_projection_norm, cfg.norm_eps)
    b = self.per_layer_input_embedding[t].view(*t.shape, L, P) * math.sqrt(P)
    return (a + b.to(a.dtype)) * (2.0 ** -0.5)

  def decode(self, x):
    return F.linear(x, self.input_embedding)


class Gemma4(nn.Module):
  """Text-only Gemma 4. Call contract of the other families:
  `(tokens, positions, cache, attention_mask, skip_lm_head=False) -> (logits fp32 | hidden, new_cache)`."""

  def __init__(self, config: ModelConfig, device=None):
    super().__init__()
    self.config = config
    types = config.attention_types()
    self.kv_sharing = kv_sharing_pattern(config.num_layers, config.frac_shared_layers, types)
    self.shared_origins = {j for i, j in enumerate(self.kv_sharing) if i != j}
    for i, j in enumerate(self.kv_sharing):
      if types[i] != types[j]:
        raise ValueError(f"layer {i} ({types[i].name}) would share the K/V of layer {j} ({types[j].name}): the "
                         "unshared part of the stack must end with a local layer followed by a global one")
    self.embedder = Embedder(config, device)
    layers = []
    for i, t in enumerate(types):
      shared = self.kv_sharing[i] != i
      hidden = config.override_kv_shared_ffw_hidden if (shared and config.override_kv_shared_ffw_hidden) \
          else config.hidden_dim
      layers.append(DecoderLayer(config, t, hidden, owns_kv=not shared, device=device))
    self.layers = nn.ModuleList(layers)
    self.final_norm = _param(config.embed_dim, ones=True, dtype=config.dtype, device=device)
    if config.vision_encoder is not None:
      from . import vision
      self.vision_encoder = vision.VisionEncoder(config.vision_encoder, dtype=config.dtype, device=device)
    if config.audio_encoder is not None:
      from . import audio
      self.audio_encoder = audio.AudioTokenizer(config.audio_encoder, dtype=config.dtype, device=device)

  def init_weights(self, seed: int = 0, scale: float = 0.02) -> "Gemma4":
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
      for n, p in self.named_parameters():
        if p.dim() >= 2:
          p.copy_((torch.randn(p.shape, generator=g) * scale).to(p.dtype))
    return self

  def head_weight(self) -> torch.Tensor:
    return self.embedder.input_embedding

  def init_cache(self, batch_size: int, cache_size: int, dtype=None, device=None) -> Dict[str, Dict[str, torch.Tensor]]:
    dtype = dtype or self.config.dtype
    device = device or self.final_norm.device
    cache = {}
    for i, layer in enumerate(self.layers):
      if self.kv_sharing[i] != i:
        continue
      a = layer.attn
      length = cache_size
      if (self.config.use_sliding_window_kv_cache and a.attn_type == AttentionType.LOCAL_SLIDING
          and self.config.sliding_window_size):
        length = min(cache_size, self.config.sliding_window_size)
      shape = (batch_size, length, a.num_kv_heads, a.head_dim)
      cache[f"layer_{i}"] = {"k": torch.zeros(shape, dtype=dtype, device=device),
                             "v": torch.zeros(shape, dtype=dtype, device=device),
                             "end_index": torch.zeros(batch_size, dtype=torch.long, device=device)}
    return cache

  def compute_final_logits(self, hidden: torch.Tensor) -> torch.Tensor:
    logits = self.embedder.decode(hidden).float()
    cap = self.config.final_logit_softcap
    return torch.tanh(logits / cap) * cap if cap else logits

  def _merge_modalities(self, x, tokens, images, audios):
    """Overwrites the embeddings at image / audio placeholder tokens with the towers' soft tokens."""
    from . import vision as vision_lib
    if images is not None and self.config.vision_encoder is not None:
      soft = vision_lib.soft_tokens_per_row(self.vision_encoder, images)
      if soft is not None:
        x = vision_lib.merge_soft_tokens(x, self.embedder.encode_vision(soft), tokens == IMAGE_SOFT_TOKEN_PLACEHOLDER)
    if audios is not None and self.config.audio_encoder is not None:
      from . import audio as audio_lib
      soft = audio_lib.soft_tokens_per_row(self.audio_encoder, audios)
      if soft is not None:
        x = vision_lib.merge_soft_tokens(x, self.embedder.encode_audio(soft), tokens == AUDIO_SOFT_TOKEN_PLACEHOLDER)
    return x

  def forward(self, input_tokens, positions=None, cache=None, attention_mask=None, output_hidden_states: bool = False,
              segment_ids=None, skip_lm_head: bool = False, images=None, audios=None):
    del output_hidden_states, segment_ids
    B, T = input_tokens.shape
    if positions is None:
      positions = torch.arange(T, device=input_tokens.device)[None].expand(B, T)
    x = self.embedder.encode(input_tokens)
    x = self._merge_modalities(x, input_tokens, images, audios)
    local_mask = attention_mask
    if (T > 1 and images is not None and attention_mask is not None
        and self.config.use_bidirectional_attention == "vision"):
      local_mask = add_bidirectional_blocks(attention_mask, input_tokens == IMAGE_SOFT_TOKEN_PLACEHOLDER)
    per_layer = self.embedder.encode_per_layer_input(x, input_tokens) if self.config.per_layer_input_dim > 0 else None
    new_cache = {} if cache is not None else None
    fresh: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    for i, layer in enumerate(self.layers):
      origin = self.kv_sharing[i]
      shared = origin != i
      ring_prefill = (cache is not None and T > 1 and self.config.use_sliding_window_kv_cache
                      and layer.attn.attn_type == AttentionType.LOCAL_SLIDING and bool(self.config.sliding_window_size))
      if shared:
        # with a cache the origin layer's updated cache holds all keys so far; without one - or while a prompt is
        # prefilled into a window-sized ring, which cannot hold it - this call's own keys
        if cache is not None and not ring_prefill:
          oc = new_cache[f"layer_{origin}"]
          shared_kv = {"k": oc["k"], "v": oc["v"], "end_index": oc["end_index"]}
        else:
          shared_kv = {"k": fresh[origin][0], "v": fresh[origin][1]}
        layer_cache = None
      else:
        shared_kv = None
        layer_cache = cache[f"layer_{i}"] if cache is not None else None
      lc, x, kv = layer(x, positions, layer_cache,
                        local_mask if layer.attn.attn_type == AttentionType.LOCAL_SLIDING else attention_mask,
                        per_layer[:, :, i, :] if per_layer is not None else None, shared_kv,
                        slot_keys=cache is not None and not ring_prefill)
      if i in self.shared_origins and (cache is None or ring_prefill):
        fresh[i] = kv
      if not shared and new_cache is not None:
        new_cache[f"layer_{i}"] = lc
    x = rms(x, self.final_norm, self.config.norm_eps)
    if skip_lm_head:
      return x, new_cache
    return self.compute_final_logits(x), new_cache
