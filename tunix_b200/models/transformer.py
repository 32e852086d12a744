"""One decoder implementation for every model family.

The reference keeps a separate module tree per family (tunix/models/{gemma,gemma3,llama3,
qwen2,qwen3}/model.py). They differ only in a handful of switches - norm flavour, q/k-norm,
biases, activation, soft-caps, sliding windows, post-norms, MoE - so here a single
`Transformer` is driven by a `ModelConfig`; each family package contributes presets, its
Hugging Face key map and its checkpoint-tree names.

Call contract (same as the reference, tunix/models/qwen3/model.py:1268-1356):

    logits_or_hidden, new_cache = model(input_tokens[B,L], positions[B,L], cache | None,
                                        attention_mask[B,L,S] | None, output_hidden_states=False,
                                        segment_ids=None, skip_lm_head=False)

`attention_mask=None` means plain causal attention over unpadded rows and unlocks the flash
kernels; a boolean tensor is honoured exactly.

Weights are stored GEMM-ready: `[out, in]` with q/k/v and gate/up projections fused, which is
also the Hugging Face layout (no transposes at import). `tunix_b200.ckpt.layout` maps these to
the reference's `[D,N,H]`-style trees for Orbax-compatible checkpoints.
"""
from __future__ import annotations

import dataclasses
import enum
import math
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.utils.checkpoint as torch_ckpt

from ..ops import functional as F
from ..ops import ref as R

Cache = Dict[str, Dict[str, torch.Tensor]]


class RematConfig(enum.Enum):
  NONE = enum.auto()      # keep all activations
  BLOCK = enum.auto()     # recompute each decoder layer in backward
  DECODER = enum.auto()   # recompute the whole stack in backward


class AttentionType(enum.Enum):
  GLOBAL = 1
  LOCAL_SLIDING = 2


@dataclasses.dataclass
class ModelConfig:
  """Architecture switches shared by all families."""

  num_layers: int
  vocab_size: int
  embed_dim: int
  hidden_dim: int
  num_heads: int
  head_dim: int
  num_kv_heads: int
  rope_theta: float = 10_000.0
  norm_eps: float = 1e-6
  # family switches
  weight_tying: bool = False             # lm_head shares the embedding table
  use_qk_norm: bool = False              # per-head RMSNorm on q and k before RoPE (Qwen3, Gemma3)
  qkv_bias: bool = False                 # Qwen2
  activation: str = "silu"               # "silu" (SwiGLU) or "gelu" (GeGLU, tanh approximation)
  norm_offset: float = 0.0               # Gemma: scale = 1 + w
  embed_scale: bool = False              # Gemma: embeddings * sqrt(D)
  attn_logits_soft_cap: Optional[float] = None
  final_logit_softcap: Optional[float] = None
  sliding_window_size: Optional[int] = None
  attention_types: Optional[Sequence[AttentionType]] = None   # pattern repeated over layers
  use_post_attn_norm: bool = False
  use_post_ffw_norm: bool = False
  local_rope_theta: Optional[float] = None
  rope_scale_factor: float = 1.0         # global-layer RoPE position scale (Gemma3 >= 4b: 8)
  query_pre_attn_scalar: Optional[float] = None
  # mixture of experts (Qwen3-MoE): softmax router -> top-k -> optional renormalise
  num_experts: int = 0
  num_experts_per_tok: int = 0
  moe_hidden_dim: int = 0
  norm_topk_prob: bool = True
  # execution
  remat_config: RematConfig = RematConfig.NONE
  dtype: torch.dtype = torch.float32
  family: str = "generic"
  max_position: int = 0                   # hint for the RoPE table (0 = grow on demand)
  fused_layers: bool = True               # training fast path: one autograd node per layer

  @property
  def is_moe(self) -> bool:
    return self.num_experts > 0

  @property
  def attn_scale(self) -> float:
    return (self.query_pre_attn_scalar or self.head_dim) ** -0.5

  def layer_attention_type(self, i: int) -> AttentionType:
    if not self.attention_types:
      return AttentionType.GLOBAL
    return self.attention_types[i % len(self.attention_types)]

  def replace(self, **kw) -> "ModelConfig":
    return dataclasses.replace(self, **kw)


def _param(*shape, dtype, device=None) -> nn.Parameter:
  return nn.Parameter(torch.empty(*shape, dtype=dtype, device=device))


class RMSNorm(nn.Module):

  def __init__(self, dim: int, eps: float, offset: float, dtype, device=None):
    super().__init__()
    self.w = _param(dim, dtype=dtype, device=device)
    self.eps, self.offset = eps, offset

  def forward(self, x):
    return F.rms_norm(x, self.w, self.eps, self.offset)


class Linear(nn.Module):
  """`y = x w^T (+ b)`, weight `[out, in]`, with optional LoRA adapters on output slices.

  An adapter `name` covering output columns `[lo, hi)` contributes
  `(x A^T) B^T * alpha / rank` with `A [rank, in]`, `B [hi - lo, rank]`; several adapters can
  sit on one fused projection (q, k and v of a fused qkv weight).
  """

  def __init__(self, in_dim: int, out_dim: int, bias: bool, dtype, device=None,
               slices: Optional[Dict[str, Tuple[int, int]]] = None):
    super().__init__()
    self.in_dim, self.out_dim = in_dim, out_dim
    self.w = _param(out_dim, in_dim, dtype=dtype, device=device)
    self.b = _param(out_dim, dtype=dtype, device=device) if bias else None
    self.slices = slices or {"": (0, out_dim)}
    self.lora_a = nn.ParameterDict()
    self.lora_b = nn.ParameterDict()
    self.lora_scale: Dict[str, float] = {}
    self.quant = None   # set by qlora: NF4-packed frozen weight replacing `w`

  def weight(self) -> torch.Tensor:
    if self.quant is not None:
      return self.quant.dequantize()
    return self.w

  def add_lora(self, name: str, rank: int, alpha: float, dtype=None, device=None) -> None:
    lo, hi = self.slices[name]
    dtype = dtype or self.w.dtype
    device = device or self.w.device
    key = name or "w"
    a = nn.Parameter(torch.empty(rank, self.in_dim, dtype=dtype, device=device))
    b = nn.Parameter(torch.zeros(hi - lo, rank, dtype=dtype, device=device))
    nn.init.kaiming_uniform_(a.data.float(), a=math.sqrt(5))
    a.data.copy_(nn.init.kaiming_uniform_(torch.empty(rank, self.in_dim), a=math.sqrt(5)).to(dtype))
    a.is_lora = True
    b.is_lora = True
    self.lora_a[key] = a
    self.lora_b[key] = b
    self.lora_scale[key] = alpha / rank

  def _adapters(self):
    out = []
    for key, a in self.lora_a.items():
      lo, hi = self.slices["" if key == "w" else key]
      out.append((a, self.lora_b[key], self.lora_scale[key], lo, hi))
    return out

  def _lora_active(self) -> bool:
    # adapters whose scale was zeroed (reference pass over a shared backbone) cost nothing
    return len(self.lora_a) > 0 and any(v != 0 for v in self.lora_scale.values())

  def forward(self, x):
    if not self._lora_active():
      return F.linear(x, self.weight(), self.b)
    if self.quant is None and self.b is None and x.is_cuda:
      from ..ops import lora as lora_ops
      adapters = self._adapters()
      if lora_ops.supported(x.reshape(-1, x.shape[-1]), self.w, adapters):
        return lora_ops.fused_lora_linear(x, self.w, adapters)      # adapter folded into the base GEMM
    y = F.linear(x, self.weight(), self.b)
    if len(self.lora_a):
      for key, a in self.lora_a.items():
        lo, hi = self.slices["" if key == "w" else key]
        t = F.linear(x, a)
        d = F.linear(t, self.lora_b[key]) * self.lora_scale[key]
        if lo == 0 and hi == self.out_dim:
          y = y + d
        else:
          y = torch.cat([y[..., :lo], y[..., lo:hi] + d, y[..., hi:]], dim=-1)
    return y


class Embedder(nn.Module):

  def __init__(self, vocab: int, dim: int, scale: bool, dtype, device=None):
    super().__init__()
    self.input_embedding = _param(vocab, dim, dtype=dtype, device=device)
    self.scale = math.sqrt(dim) if scale else 1.0

  def encode(self, tokens):
    return F.embedding(tokens, self.input_embedding, self.scale)


class Attention(nn.Module):

  def __init__(self, cfg: ModelConfig, layer_idx: int, device=None):
    super().__init__()
    self.cfg = cfg
    N, K, H, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.embed_dim
    self.attn_type = cfg.layer_attention_type(layer_idx)
    slices = {"q_proj": (0, N * H), "k_proj": (N * H, (N + K) * H), "v_proj": ((N + K) * H, (N + 2 * K) * H)}
    self.qkv_proj = Linear(D, (N + 2 * K) * H, cfg.qkv_bias, cfg.dtype, device, slices)
    self.o_proj = Linear(N * H, D, False, cfg.dtype, device, {"o_proj": (0, D)})
    if cfg.use_qk_norm:
      self.q_norm = RMSNorm(H, cfg.norm_eps, cfg.norm_offset, cfg.dtype, device)
      self.k_norm = RMSNorm(H, cfg.norm_eps, cfg.norm_offset, cfg.dtype, device)
    else:
      self.q_norm = self.k_norm = None

  def _forward_paged(self, q, k, v, cache, B, T):
    return _paged_attention(self, q, k, v, cache, B, T)

  def _theta_scale(self) -> Tuple[float, float]:
    cfg = self.cfg
    if self.attn_type == AttentionType.LOCAL_SLIDING and cfg.local_rope_theta:
      return cfg.local_rope_theta, 1.0
    return cfg.rope_theta, cfg.rope_scale_factor

  def forward(self, x, positions, cache, attn_mask, layer_name: str):
    cfg = self.cfg
    B, T, _ = x.shape
    N, K, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
    qkv = self.qkv_proj(x)
    theta, rscale = self._theta_scale()
    qkv = F.qk_norm_rope(qkv, positions, N, K, H, theta,
                         self.q_norm.w if self.q_norm is not None else None,
                         self.k_norm.w if self.k_norm is not None else None,
                         cfg.norm_eps, cfg.norm_offset, rscale, cfg.max_position)
    qkv = qkv.view(B, T, N + 2 * K, H)
    q, k, v = qkv[:, :, :N], qkv[:, :, N:N + K], qkv[:, :, N + K:]

    if cache is not None and not isinstance(cache, dict):
      return self._forward_paged(q, k, v, cache, B, T)

    new_cache = None
    if cache is not None:
      ck, cv, end = cache["k"], cache["v"], cache["end_index"]
      S = ck.shape[1]
      # ring-buffer write at end_index % cache_size (tunix/models/qwen3/model.py:556-571)
      idx = (end[:, None] + torch.arange(T, device=x.device)[None, :]) % S          # [B, T]
      bidx = torch.arange(B, device=x.device)[:, None].expand(B, T)
      ck = ck.index_put((bidx, idx), k.to(ck.dtype))
      cv = cv.index_put((bidx, idx), v.to(cv.dtype))
      new_cache = {"k": ck, "v": cv, "end_index": end + T}
      k, v = ck, cv

    sp_group = getattr(self, "sp_group", None)
    if (cache is None and sp_group is None and x.is_cuda and not cfg.attn_logits_soft_cap
        and not (self.attn_type == AttentionType.LOCAL_SLIDING and cfg.sliding_window_size)):
      # plain causal (or packed-segment) attention straight from the fused q|k|v tensor: one gradient buffer
      from ..ops import attention as attn_ops, flash as flash_lib
      seg = isinstance(attn_mask, attn_ops.SegmentMask)
      if (attn_mask is None or seg) and flash_lib.packed_supported(qkv, N, K):
        o = flash_lib.flash_attention_packed(qkv, N, K, causal=True, scale=cfg.attn_scale,
                                             segments=attn_mask.bounds() if seg else None)
        return self.o_proj(o.reshape(B, T, N * H)), None
    if sp_group is not None:
      if cache is not None or attn_mask is not None:
        raise NotImplementedError("sequence parallelism covers causal training / scoring without a KV cache")
      if self.attn_type == AttentionType.LOCAL_SLIDING and cfg.sliding_window_size:
        raise NotImplementedError("sequence parallelism does not cover sliding-window layers")
      from ..dist import sp as sp_lib
      # every held query chunk attends the key prefix that ends with it (queries aligned to the end of the keys)
      o = sp_lib.attention(q, k, v, sp_group, self.sp_layout,
                           lambda qc, kc, vc: F.attention(qc, kc, vc, mask=None, causal=True, scale=cfg.attn_scale,
                                                          softcap=cfg.attn_logits_soft_cap or 0.0))
      return self.o_proj(o.reshape(B, T, N * H)), None

    mask = attn_mask
    causal = mask is None and cache is None
    if mask is not None and not isinstance(mask, torch.Tensor) and (
        cache is not None or (self.attn_type == AttentionType.LOCAL_SLIDING and cfg.sliding_window_size)):
      mask = mask.dense()
    if self.attn_type == AttentionType.LOCAL_SLIDING and cfg.sliding_window_size:
      mask = _apply_sliding_window(mask, positions, k.shape[1], cfg.sliding_window_size, cache is not None)
      causal = False
    o = F.attention(q, k, v, mask=mask, causal=causal, scale=cfg.attn_scale,
                    softcap=cfg.attn_logits_soft_cap or 0.0)
    out = self.o_proj(o.reshape(B, T, N * H))
    return out, new_cache


def _paged_attention(attn: "Attention", q, k, v, cache, B: int, T: int):
  """Paged KV cache path (`rollout.paged_cache.PagedLayerCache`): store the new K/V rows in
  their pages, then attend - within the prompt for a prefill, through the block tables for a
  decode step."""
  from ..ops import paged
  cfg = attn.cfg
  N, K, H = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
  paged.kv_page_write(k.reshape(B * T, K, H), v.reshape(B * T, K, H), cache.slots, cache.k_pages, cache.v_pages)
  if cache.mode == "decode":
    if T != 1:
      raise ValueError("a paged decode step takes one token per sequence")
    o = paged.paged_decode_attention(q.reshape(B, N, H), cache.k_pages, cache.v_pages, cache.block_tables,
                                     cache.seq_lens, cfg.attn_scale, cache.num_splits, cache.max_len)
    o = o.view(B, 1, N * H)
  else:
    o = F.attention(q, k, v, mask=None, causal=True, scale=cfg.attn_scale,
                    softcap=cfg.attn_logits_soft_cap or 0.0).reshape(B, T, N * H)
  return attn.o_proj(o), cache


def _apply_sliding_window(mask, positions, S, window, cached):
  """Restricts attention to keys within `window` positions of the query
  (tunix/models/gemma/model.py:313-339). Only defined for the non-cached, position-ordered
  layout and for caches that have not wrapped."""
  B, T = positions.shape
  dev = positions.device
  if mask is None:
    mask = torch.ones(T, S, dtype=torch.bool, device=dev).tril(S - T)[None].expand(B, T, S)
  if cached:
    # key slot index == absolute position while the ring buffer has not wrapped
    kpos = torch.arange(S, device=dev)[None, None, :]
  else:
    kpos = positions[:, None, :]
  qpos = positions[:, :, None]
  win = (kpos > qpos - window) & (kpos < qpos + window)
  return mask & win


class MLP(nn.Module):

  def __init__(self, cfg: ModelConfig, device=None):
    super().__init__()
    D, Fh = cfg.embed_dim, cfg.hidden_dim
    self.kind = cfg.activation
    self.gate_up_proj = Linear(D, 2 * Fh, False, cfg.dtype, device, {"gate_proj": (0, Fh), "up_proj": (Fh, 2 * Fh)})
    self.down_proj = Linear(Fh, D, False, cfg.dtype, device, {"down_proj": (0, D)})

  def forward(self, x):
    return self.down_proj(F.glu(self.gate_up_proj(x), self.kind))


class MoELayer(nn.Module):
  """Top-k routed experts: softmax over E router logits, top-k, optional renormalisation,
  weighted sum of SwiGLU experts (tunix/models/qwen3/model.py:744-1042). Expert weights are
  stacked: gate_up `[E, 2F, D]`, down `[E, D, F]`. Tokens are sorted by expert and each expert
  runs one GEMM chain over its contiguous rows; under expert parallelism the sorted rows are
  exchanged by `tunix_b200.dist.moe`."""

  def __init__(self, cfg: ModelConfig, device=None):
    super().__init__()
    self.cfg = cfg
    E, D, Fh = cfg.num_experts, cfg.embed_dim, cfg.moe_hidden_dim
    self.router = Linear(D, E, False, cfg.dtype, device)
    self.gate_up_proj = _param(E, 2 * Fh, D, dtype=cfg.dtype, device=device)
    self.down_proj = _param(E, D, Fh, dtype=cfg.dtype, device=device)
    self.ep_group = None   # set by dist.moe.shard_experts

  def route(self, x2):
    cfg = self.cfg
    logits = self.router(x2).float()
    probs = torch.softmax(logits, dim=-1)
    topv, topi = torch.topk(probs, cfg.num_experts_per_tok, dim=-1)
    if cfg.norm_topk_prob:
      topv = topv / topv.sum(-1, keepdim=True)
    return topv, topi

  def experts(self, xs: torch.Tensor, counts: List[int], first_expert: int = 0) -> torch.Tensor:
    """xs: rows sorted by expert; counts[e] rows belong to local expert e."""
    from ..ops import moe as moe_ops
    return moe_ops.grouped_mlp(xs, counts, self.gate_up_proj, self.down_proj, self.cfg.activation, first_expert)

  def forward(self, x):
    cfg = self.cfg
    B, T, D = x.shape
    x2 = x.reshape(B * T, D)
    topv, topi = self.route(x2)
    if self.ep_group is not None:
      from ..dist import moe as dist_moe
      y = dist_moe.ep_forward(self, x2, topv, topi)
      return y.view(B, T, D)
    from ..ops import moe as moe_ops
    if moe_ops.grouped_supported(x2, self.gate_up_proj) and moe_ops.grouped_supported(x2, self.down_proj):
      # one grouped tensor-core launch per projection, routing kept on the device
      y = moe_ops.moe_forward_padded(x2, topv, topi, self.gate_up_proj, self.down_proj, cfg.activation)
      return y.view(B, T, D)
    k = cfg.num_experts_per_tok
    flat_e = topi.reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    tok = order // k
    xs = x2.index_select(0, tok)
    counts = torch.bincount(flat_e, minlength=cfg.num_experts).tolist()
    ys = self.experts(xs, counts)
    w = topv.reshape(-1).index_select(0, order).to(ys.dtype)
    y = torch.zeros_like(x2).index_add_(0, tok, ys * w[:, None])
    return y.view(B, T, D)


class DecoderLayer(nn.Module):

  def __init__(self, cfg: ModelConfig, layer_idx: int, device=None):
    super().__init__()
    self.cfg = cfg
    mk = lambda: RMSNorm(cfg.embed_dim, cfg.norm_eps, cfg.norm_offset, cfg.dtype, device)
    self.input_layernorm = mk()
    self.attn = Attention(cfg, layer_idx, device)
    self.post_attention_layernorm = mk()     # the pre-MLP norm
    self.post_attn_norm = mk() if cfg.use_post_attn_norm else None
    self.post_ffw_norm = mk() if cfg.use_post_ffw_norm else None
    self.mlp = MoELayer(cfg, device) if cfg.is_moe else MLP(cfg, device)

  def forward(self, h, positions, cache, attn_mask, layer_name=""):
    if self.cfg.fused_layers and torch.is_grad_enabled():
      from ..ops import fused_layer
      if fused_layer.eligible(self, h, cache, attn_mask):
        return fused_layer.run(self, h, positions, attn_mask), None
    if cache is not None and not isinstance(cache, dict) and not torch.is_grad_enabled():
      from ..ops import decode_layer
      if decode_layer.eligible(self, h, cache):      # paged decode step: eight launches per layer
        return decode_layer.run(self, h, positions, cache), cache
    x = self.input_layernorm(h)
    a, new_cache = self.attn(x, positions, cache, attn_mask, layer_name)
    if self.post_attn_norm is not None:
      a = self.post_attn_norm(a)
    # residual add fused with the pre-MLP norm
    x, h = F.add_rms_norm(a, h, self.post_attention_layernorm.w, self.cfg.norm_eps, self.cfg.norm_offset)
    m = self.mlp(x)
    if self.post_ffw_norm is not None:
      m = self.post_ffw_norm(m)
    return h + m, new_cache


class Transformer(nn.Module):
  """Decoder-only LM."""

  def __init__(self, config: ModelConfig, device=None):
    super().__init__()
    self.config = config
    self.embedder = Embedder(config.vocab_size, config.embed_dim, config.embed_scale, config.dtype, device)
    self.layers = nn.ModuleList([DecoderLayer(config, i, device) for i in range(config.num_layers)])
    self.final_norm = RMSNorm(config.embed_dim, config.norm_eps, config.norm_offset, config.dtype, device)
    if config.weight_tying:
      self.lm_head = None
    else:
      self.lm_head = Linear(config.embed_dim, config.vocab_size, False, config.dtype, device)

  # ---- reference API ---------------------------------------------------------------
  @property
  def num_embed(self) -> int:
    return self.config.vocab_size

  def head_weight(self) -> torch.Tensor:
    """[V, D] matrix of the output projection (the embedding table when tied)."""
    return self.embedder.input_embedding if self.lm_head is None else self.lm_head.weight()

  def init_cache(self, batch_size: int, cache_size: int, dtype: Optional[torch.dtype] = None, device=None) -> Cache:
    cfg = self.config
    dtype = dtype or cfg.dtype
    device = device or self.embedder.input_embedding.device
    return {
        f"layer_{i}": {
            "k": torch.zeros(batch_size, cache_size, cfg.num_kv_heads, cfg.head_dim, dtype=dtype, device=device),
            "v": torch.zeros(batch_size, cache_size, cfg.num_kv_heads, cfg.head_dim, dtype=dtype, device=device),
            "end_index": torch.zeros(batch_size, dtype=torch.long, device=device),
        } for i in range(cfg.num_layers)
    }

  def get_model_input(self) -> Dict[str, torch.Tensor]:
    """Dummy inputs with the shapes `__call__` expects."""
    dev = self.embedder.input_embedding.device
    B, L = 2, 1
    return {
        "input_tokens": torch.ones(B, L, dtype=torch.long, device=dev),
        "positions": torch.ones(B, L, dtype=torch.long, device=dev),
        "cache": None,
        "attention_mask": torch.ones(B, 1, L, dtype=torch.bool, device=dev),
    }

  def compute_final_logits(self, hidden: torch.Tensor, as_float: bool = True) -> torch.Tensor:
    """lm_head (or tied `h E^T`) in fp32, with the final soft-cap when configured.

    `as_float=False` returns the GEMM's own dtype when no soft-cap applies: the sampler kernel
    reads bf16 rows directly, which saves a pass over [B, V] per decode step."""
    w = self.head_weight()
    if getattr(self, "tp_size", 1) > 1 and getattr(w, "vocab_parallel", None) is None:
      # a replicated head on tensor-parallel ranks: every rank must get the same bits, or the ranks of a
      # group would sample different tokens - no reduction whose order varies from run to run
      from ..ops import kernels
      with kernels.fixed_reduction_order():
        logits = F.linear(hidden, w)
    else:
      logits = F.linear(hidden, w)
    vp = getattr(w, "vocab_parallel", None)
    if vp is not None:       # vocabulary-parallel head: every rank computed its slice of the logits
      import torch.distributed as dist
      parts = [torch.empty_like(logits) for _ in range(dist.get_world_size(vp[0]))]
      dist.all_gather(parts, logits.contiguous(), group=vp[0])
      logits = torch.cat(parts, dim=-1)
    cap = self.config.final_logit_softcap
    if cap:
      logits = logits.float()
      logits = torch.tanh(logits / cap) * cap
    elif as_float:
      logits = logits.float()
    return logits

  def _stack(self, h, positions, cache, attn_mask):
    new_cache = {} if cache is not None else None
    use_block_remat = (self.config.remat_config == RematConfig.BLOCK and torch.is_grad_enabled() and cache is None)
    for i, layer in enumerate(self.layers):
      name = f"layer_{i}"
      lc = cache[name] if cache is not None else None
      if use_block_remat:
        h, _ = torch_ckpt.checkpoint(layer, h, positions, None, attn_mask, name, use_reentrant=False)
      else:
        h, nc = layer(h, positions, lc, attn_mask, name)
        if new_cache is not None:
          new_cache[name] = nc
    return h, new_cache

  def forward(self, input_tokens, positions=None, cache: Optional[Cache] = None, attention_mask=None,
              output_hidden_states: bool = False, segment_ids=None, skip_lm_head: bool = False,
              input_embeddings: Optional[torch.Tensor] = None):
    """`input_embeddings` [B, L, D] replaces the embedding lookup (multimodal models merge image or audio
    soft tokens into the text embeddings first); `input_tokens` then only gives the shape."""
    cfg = self.config
    B, L = input_tokens.shape
    if positions is None:
      positions = torch.arange(L, device=input_tokens.device)[None].expand(B, L)
    if segment_ids is not None:
      from ..ops import attention as attn_ops
      seg_mask = attn_ops.SegmentMask(segment_ids)      # symbolic: the flash kernels take segment bounds
      attention_mask = seg_mask if attention_mask is None else (attention_mask & seg_mask.dense())
    h = self.embedder.encode(input_tokens) if input_embeddings is None else input_embeddings
    if cfg.remat_config == RematConfig.DECODER and torch.is_grad_enabled() and cache is None:
      h = torch_ckpt.checkpoint(lambda hh: self._stack(hh, positions, None, attention_mask)[0], h, use_reentrant=False)
      new_cache = None
    else:
      h, new_cache = self._stack(h, positions, cache, attention_mask)
    h = self.final_norm(h)
    self.last_hidden_state = h if output_hidden_states else None
    if skip_lm_head:
      return h, new_cache
    return self.compute_final_logits(h), new_cache

  # ---- initialisation ----------------------------------------------------------------
  @torch.no_grad()
  def init_weights(self, seed: int = 0, scale: float = 0.02) -> "Transformer":
    """N(0, scale) for matrices, unit norms (zero for Gemma's 1+w form), zero biases
    (tunix/models/dummy_model_creator.py:30-92)."""
    gens: Dict[str, torch.Generator] = {}
    for name, p in self.named_parameters():
      dev = str(p.device)
      if dev not in gens:
        g = torch.Generator(device=p.device)
        g.manual_seed(seed)
        gens[dev] = g
      if getattr(p, "is_lora", False):
        continue
      if p.dim() >= 2:
        if p.dtype == torch.float32 or p.device.type == "cuda":
          p.normal_(0.0, scale, generator=gens[dev])
        else:
          p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, scale, generator=gens[dev]))
      elif name.endswith(".b"):
        p.zero_()
      else:
        p.fill_(0.0 if self.config.norm_offset == 1.0 else 1.0)
    return self


def num_params(cfg: ModelConfig) -> int:
  """Parameter count implied by a config (no allocation)."""
  D, Fh, N, K, H, V, L = (cfg.embed_dim, cfg.hidden_dim, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim,
                          cfg.vocab_size, cfg.num_layers)
  attn = D * (N + 2 * K) * H + N * H * D + (2 * H if cfg.use_qk_norm else 0) + ((N + 2 * K) * H if cfg.qkv_bias else 0)
  if cfg.is_moe:
    mlp = D * cfg.num_experts + cfg.num_experts * 3 * D * cfg.moe_hidden_dim
  else:
    mlp = 3 * D * Fh
  norms = 2 * D + (D if cfg.use_post_attn_norm else 0) + (D if cfg.use_post_ffw_norm else 0)
  return L * (attn + mlp + norms) + V * D * (1 if cfg.weight_tying else 2) + D
