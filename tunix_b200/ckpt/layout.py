"""Module parameters <-> checkpoint trees.

Internally weights are GEMM-ready (`[out, in]`, fused q|k|v and gate|up). Checkpoints use the
reference's tree so that either framework can read the other's files
(tunix/models/qwen3/params.py:47-116, tunix/models/llama3/params.py:24-79):

  embedder.input_embedding [V,D]; layers.i.attn.{q_proj.w [D,N,H], k_proj.w / v_proj.w [D,K,H],
  o_proj.w [N,H,D], q_norm.w / k_norm.w [H]}; layers.i.mlp.{gate_proj,up_proj}.kernel [D,F],
  down_proj.kernel [F,D]; MoE router.kernel [D,E], gate_proj/up_proj [E,D,F], down_proj [E,F,D];
  layers.i.{input_layernorm,post_attention_layernorm}.w [D]; final_norm.w; lm_head.w [D,V];
  LoRA leaves `<param>_lora_a` / `<param>_lora_b` (q_proj.w_lora_a [D,r], w_lora_b [r,N,H],
  o_proj.w_lora_a [N,H,r], w_lora_b [r,D], kernel_lora_a [in,r], kernel_lora_b [r,out]).

Every leaf ends with the key "value" (the variable wrapper of the reference's module system).
Modules that are not `Transformer`s are saved under their own dotted names.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Iterable, List, Mapping, Optional, Tuple, Union

import torch

from .orbax_layout import Key, ShardedArray


def _generic_key(name: str) -> Key:
  return tuple(int(p) if p.isdigit() else p for p in name.split(".")) + ("value",)


def _is_transformer(model) -> bool:
  from ..models.transformer import Transformer
  return isinstance(model, Transformer)


def model_to_tree(model: torch.nn.Module, lora_only: bool = False) -> Dict[Key, torch.Tensor]:
  """Exports parameters in the checkpoint tree layout (tensors are views/copies on the same device)."""
  if not _is_transformer(model):
    return {_generic_key(n): p.detach() for n, p in model.named_parameters()
            if not lora_only or getattr(p, "is_lora", False)}
  cfg = model.config
  N, K, H, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.embed_dim
  out: Dict[Key, torch.Tensor] = {}

  def put(key: Key, t: torch.Tensor, is_lora: bool = False):
    if lora_only and not is_lora:
      return
    out[key + ("value",)] = t.detach()

  put(("embedder", "input_embedding"), model.embedder.input_embedding)
  for i, layer in enumerate(model.layers):
    L = ("layers", i)
    a = layer.attn
    w = a.qkv_proj.w.detach()
    put(L + ("attn", "q_proj", "w"), w[: N * H].t().reshape(D, N, H))
    put(L + ("attn", "k_proj", "w"), w[N * H:(N + K) * H].t().reshape(D, K, H))
    put(L + ("attn", "v_proj", "w"), w[(N + K) * H:].t().reshape(D, K, H))
    if a.qkv_proj.b is not None:
      b = a.qkv_proj.b.detach()
      put(L + ("attn", "q_bias"), b[: N * H].reshape(N, H))
      put(L + ("attn", "k_bias"), b[N * H:(N + K) * H].reshape(K, H))
      put(L + ("attn", "v_bias"), b[(N + K) * H:].reshape(K, H))
    put(L + ("attn", "o_proj", "w"), a.o_proj.w.detach().t().reshape(N, H, D))
    if a.q_norm is not None:
      put(L + ("attn", "q_norm", "w"), a.q_norm.w)
      put(L + ("attn", "k_norm", "w"), a.k_norm.w)
    for nm, heads in (("q_proj", N), ("k_proj", K), ("v_proj", K)):
      if nm in a.qkv_proj.lora_a:
        put(L + ("attn", nm, "w_lora_a"), a.qkv_proj.lora_a[nm].detach().t(), True)                   # [D, r]
        put(L + ("attn", nm, "w_lora_b"), a.qkv_proj.lora_b[nm].detach().t().reshape(-1, heads, H), True)  # [r,N,H]
    if "o_proj" in a.o_proj.lora_a:
      put(L + ("attn", "o_proj", "w_lora_a"), a.o_proj.lora_a["o_proj"].detach().t().reshape(N, H, -1), True)
      put(L + ("attn", "o_proj", "w_lora_b"), a.o_proj.lora_b["o_proj"].detach().t(), True)
    put(L + ("input_layernorm", "w"), layer.input_layernorm.w)
    put(L + ("post_attention_layernorm", "w"), layer.post_attention_layernorm.w)
    if layer.post_attn_norm is not None:
      put(L + ("post_attn_norm", "w"), layer.post_attn_norm.w)
    if layer.post_ffw_norm is not None:
      put(L + ("post_ffw_norm", "w"), layer.post_ffw_norm.w)
    m = layer.mlp
    if cfg.is_moe:
      Fh = cfg.moe_hidden_dim
      put(L + ("mlp", "router", "kernel"), m.router.w.detach().t())
      gu = m.gate_up_proj.detach()
      experts = {"gate_proj": gu[:, :Fh].transpose(1, 2), "up_proj": gu[:, Fh:].transpose(1, 2),
                 "down_proj": m.down_proj.detach().transpose(1, 2)}
      ep = getattr(m, "ep_size", 1) if getattr(m, "ep_group", None) is not None else 1
      for nm, t in experts.items():
        if ep > 1 and not lora_only:
          # this rank holds experts [ep_rank * E/ep, (ep_rank + 1) * E/ep): one chunk of the [E, ...] array
          t = t.contiguous()
          out[L + ("mlp", nm, "value")] = ShardedArray(t, (cfg.num_experts,) + tuple(t.shape[1:]), tuple(t.shape),
                                                       (m.ep_rank,) + (0,) * (t.dim() - 1))
        else:
          put(L + ("mlp", nm), t)
    else:
      Fh = cfg.hidden_dim
      gu = m.gate_up_proj.w.detach()
      put(L + ("mlp", "gate_proj", "kernel"), gu[:Fh].t())
      put(L + ("mlp", "up_proj", "kernel"), gu[Fh:].t())
      put(L + ("mlp", "down_proj", "kernel"), m.down_proj.w.detach().t())
      for nm in ("gate_proj", "up_proj"):
        if nm in m.gate_up_proj.lora_a:
          put(L + ("mlp", nm, "kernel_lora_a"), m.gate_up_proj.lora_a[nm].detach().t(), True)
          put(L + ("mlp", nm, "kernel_lora_b"), m.gate_up_proj.lora_b[nm].detach().t(), True)
      if "down_proj" in m.down_proj.lora_a:
        put(L + ("mlp", "down_proj", "kernel_lora_a"), m.down_proj.lora_a["down_proj"].detach().t(), True)
        put(L + ("mlp", "down_proj", "kernel_lora_b"), m.down_proj.lora_b["down_proj"].detach().t(), True)
  put(("final_norm", "w"), model.final_norm.w)
  if model.lm_head is not None:
    put(("lm_head", "w"), model.lm_head.w.detach().t())
  return out


def expected_keys(model: torch.nn.Module, lora_only: bool = False) -> List[Key]:
  return list(model_to_tree(model, lora_only).keys())


@torch.no_grad()
def tree_to_model(model: torch.nn.Module, tree: Mapping[Key, torch.Tensor], lora_only: bool = False,
                  strict: bool = True) -> None:
  """Loads a checkpoint tree into the module's parameters (in place)."""
  if not _is_transformer(model):
    for n, p in model.named_parameters():
      if lora_only and not getattr(p, "is_lora", False):
        continue
      k = _generic_key(n)
      if k not in tree:
        if strict:
          raise KeyError(f"{k} missing from checkpoint")
        continue
      p.copy_(tree[k].to(p.device, p.dtype).reshape(p.shape))
    return
  cfg = model.config
  N, K, H, D = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.embed_dim

  def get(key: Key, is_lora: bool = False) -> Optional[torch.Tensor]:
    if lora_only and not is_lora:
      return None
    k = key + ("value",)
    if k not in tree:
      if strict:
        raise KeyError(f"{k} missing from checkpoint")
      return None
    return tree[k]

  def assign(p: torch.Tensor, t: Optional[torch.Tensor]):
    if t is not None:
      p.copy_(t.to(p.device, p.dtype).reshape(p.shape))

  assign(model.embedder.input_embedding, get(("embedder", "input_embedding")))
  for i, layer in enumerate(model.layers):
    L = ("layers", i)
    a = layer.attn
    q, k, v = get(L + ("attn", "q_proj", "w")), get(L + ("attn", "k_proj", "w")), get(L + ("attn", "v_proj", "w"))
    if q is not None:
      w = a.qkv_proj.w
      w[: N * H].copy_(q.reshape(D, N * H).t().to(w.device, w.dtype))
      w[N * H:(N + K) * H].copy_(k.reshape(D, K * H).t().to(w.device, w.dtype))
      w[(N + K) * H:].copy_(v.reshape(D, K * H).t().to(w.device, w.dtype))
    if a.qkv_proj.b is not None:
      qb, kb, vb = get(L + ("attn", "q_bias")), get(L + ("attn", "k_bias")), get(L + ("attn", "v_bias"))
      if qb is not None:
        a.qkv_proj.b.copy_(torch.cat([qb.reshape(-1), kb.reshape(-1), vb.reshape(-1)]).to(a.qkv_proj.b))
    o = get(L + ("attn", "o_proj", "w"))
    if o is not None:
      assign(a.o_proj.w, o.reshape(N * H, D).t())
    if a.q_norm is not None:
      assign(a.q_norm.w, get(L + ("attn", "q_norm", "w")))
      assign(a.k_norm.w, get(L + ("attn", "k_norm", "w")))
    for nm in ("q_proj", "k_proj", "v_proj"):
      if nm in a.qkv_proj.lora_a:
        la, lb = get(L + ("attn", nm, "w_lora_a"), True), get(L + ("attn", nm, "w_lora_b"), True)
        if la is not None:
          assign(a.qkv_proj.lora_a[nm], la.t())
          assign(a.qkv_proj.lora_b[nm], lb.reshape(lb.shape[0], -1).t())
    if "o_proj" in a.o_proj.lora_a:
      la, lb = get(L + ("attn", "o_proj", "w_lora_a"), True), get(L + ("attn", "o_proj", "w_lora_b"), True)
      if la is not None:
        assign(a.o_proj.lora_a["o_proj"], la.reshape(N * H, -1).t())
        assign(a.o_proj.lora_b["o_proj"], lb.t())
    assign(layer.input_layernorm.w, get(L + ("input_layernorm", "w")))
    assign(layer.post_attention_layernorm.w, get(L + ("post_attention_layernorm", "w")))
    if layer.post_attn_norm is not None:
      assign(layer.post_attn_norm.w, get(L + ("post_attn_norm", "w")))
    if layer.post_ffw_norm is not None:
      assign(layer.post_ffw_norm.w, get(L + ("post_ffw_norm", "w")))
    m = layer.mlp
    if cfg.is_moe:
      Fh = cfg.moe_hidden_dim
      r = get(L + ("mlp", "router", "kernel"))
      if r is not None:
        assign(m.router.w, r.t())
        g, u, d = get(L + ("mlp", "gate_proj")), get(L + ("mlp", "up_proj")), get(L + ("mlp", "down_proj"))
        if getattr(m, "ep_group", None) is not None and g.shape[0] != m.gate_up_proj.shape[0]:
          per = m.gate_up_proj.shape[0]        # expert parallel: keep this rank's experts of the full arrays
          g, u, d = (t[m.ep_rank * per:(m.ep_rank + 1) * per] for t in (g, u, d))
        m.gate_up_proj[:, :Fh].copy_(g.transpose(1, 2).to(m.gate_up_proj))
        m.gate_up_proj[:, Fh:].copy_(u.transpose(1, 2).to(m.gate_up_proj))
        m.down_proj.copy_(d.transpose(1, 2).to(m.down_proj))
    else:
      Fh = cfg.hidden_dim
      g = get(L + ("mlp", "gate_proj", "kernel"))
      if g is not None:
        u, d = get(L + ("mlp", "up_proj", "kernel")), get(L + ("mlp", "down_proj", "kernel"))
        w = m.gate_up_proj.w
        w[:Fh].copy_(g.t().to(w.device, w.dtype))
        w[Fh:].copy_(u.t().to(w.device, w.dtype))
        assign(m.down_proj.w, d.t())
      for nm in ("gate_proj", "up_proj"):
        if nm in m.gate_up_proj.lora_a:
          la, lb = get(L + ("mlp", nm, "kernel_lora_a"), True), get(L + ("mlp", nm, "kernel_lora_b"), True)
          if la is not None:
            assign(m.gate_up_proj.lora_a[nm], la.t())
            assign(m.gate_up_proj.lora_b[nm], lb.t())
      if "down_proj" in m.down_proj.lora_a:
        la = get(L + ("mlp", "down_proj", "kernel_lora_a"), True)
        lb = get(L + ("mlp", "down_proj", "kernel_lora_b"), True)
        if la is not None:
          assign(m.down_proj.lora_a["down_proj"], la.t())
          assign(m.down_proj.lora_b["down_proj"], lb.t())
  assign(model.final_norm.w, get(("final_norm", "w")))
  if model.lm_head is not None:
    h = get(("lm_head", "w"))
    if h is not None:
      assign(model.lm_head.w, h.t())


# ---- optimizer state --------------------------------------------------------------------
def opt_state_to_tree(opt_state: Mapping[str, Any]) -> Dict[Key, torch.Tensor]:
  """{'count': t, 'mu': {param_name: t}, 'hyperparams': {...}} -> flat keyed tree. Parameter
  names are split on dots so the optimizer tree mirrors the module tree, as an optax state does."""
  out: Dict[Key, torch.Tensor] = {}
  for k, v in opt_state.items():
    if isinstance(v, Mapping):
      for n, t in v.items():
        out[(k,) + tuple(int(p) if p.isdigit() else p for p in str(n).split(".")) + ("value",)] = t.detach()
    else:
      out[(k, "value")] = torch.as_tensor(v).detach()
  return out


@torch.no_grad()
def tree_to_opt_state(opt_state: Dict[str, Any], tree: Mapping[Key, torch.Tensor]) -> None:
  for k, v in list(opt_state.items()):
    if isinstance(v, dict):
      for n, t in v.items():
        key = (k,) + tuple(int(p) if p.isdigit() else p for p in str(n).split(".")) + ("value",)
        if key in tree:
          if isinstance(t, torch.Tensor) and t.dim() > 0:
            t.copy_(tree[key].to(t.device, t.dtype).reshape(t.shape))
          else:
            v[n] = tree[key].to(torch.as_tensor(t).dtype)
    else:
      key = (k, "value")
      if key in tree:
        opt_state[k] = tree[key].to(torch.as_tensor(v).dtype).reshape(torch.as_tensor(v).shape)
