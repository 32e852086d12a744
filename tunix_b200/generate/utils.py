"""Helpers of the generation stack: attention masks for prefill / decode against a fixed-size
cache, padding and EOS searches, and the weight-transfer machinery used when trainer weights
are pushed into a rollout engine (tunix/generate/utils.py:34-1966)."""
from __future__ import annotations

import re
from typing import Any, Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch


def next_power_of_2(x: int) -> int:
  if x <= 0:
    return 1
  return 1 << (int(x) - 1).bit_length()


def make_prefill_attention_mask(valid: torch.Tensor, cache_size: int) -> torch.Tensor:
  """valid [B, P] -> [B, P, cache_size] causal mask over cache slots (slot j holds prompt column j)."""
  B, P = valid.shape
  causal = torch.ones(P, P, dtype=torch.bool, device=valid.device).tril()
  m = valid[:, None, :] & causal[None]
  out = torch.zeros(B, P, cache_size, dtype=torch.bool, device=valid.device)
  out[:, :, :P] = m
  return out


def make_decode_attention_mask(valid: torch.Tensor, step: int, cache_size: int) -> torch.Tensor:
  """Mask [B, 1, cache_size] for the token at buffer index `step`: slots 0..step that hold real tokens."""
  B = valid.shape[0]
  out = torch.zeros(B, 1, cache_size, dtype=torch.bool, device=valid.device)
  out[:, 0, :step + 1] = valid[:, :step + 1]
  return out


def np_find_first_non_pad_idx(ids: np.ndarray, pad_id: int) -> int:
  nz = np.nonzero(ids != pad_id)[0]
  return int(nz[0]) if len(nz) else 0


def np_find_first_eos_idx(ids: np.ndarray, eos_ids: Sequence[int]) -> int:
  """Index of the first EOS (exclusive end of the completion); len(ids) when there is none."""
  hit = np.nonzero(np.isin(ids, np.asarray(list(eos_ids))))[0]
  return int(hit[0]) if len(hit) else len(ids)


def find_first_eos_idx(ids: torch.Tensor, eos_ids: Sequence[int]) -> int:
  return np_find_first_eos_idx(ids.cpu().numpy(), eos_ids)


def pad_to_length(x: np.ndarray, target: int, pad_value=0, left: bool = False, axis: int = 0) -> np.ndarray:
  n = x.shape[axis]
  if n >= target:
    return x
  shape = list(x.shape)
  shape[axis] = target - n
  pad = np.full(shape, pad_value, dtype=x.dtype)
  return np.concatenate([pad, x] if left else [x, pad], axis=axis)


def padded_fill_tokens_and_logits(token_buffers: np.ndarray, logits_buffers, return_logits: bool, echo: bool,
                                  pad_id: int, eos_ids: Sequence[int], max_prompt_length: int, max_len: int):
  """-> (lengths [B], tokens [B, max_len] right-padded, logits or None)."""
  B = token_buffers.shape[0]
  out = np.full((B, max_len), pad_id, dtype=token_buffers.dtype)
  lengths = np.zeros(B, dtype=np.int32)
  out_logits = None
  if return_logits and logits_buffers is not None:
    out_logits = np.zeros((B, max_len) + tuple(logits_buffers.shape[2:]), dtype=np.float32)
  for i in range(B):
    start = np_find_first_non_pad_idx(token_buffers[i], pad_id) if echo else max_prompt_length
    end = np_find_first_eos_idx(token_buffers[i][max_prompt_length:], eos_ids) + max_prompt_length
    n = end - start
    lengths[i] = n
    out[i, :n] = token_buffers[i][start:end]
    if out_logits is not None:
      out_logits[i, :n] = np.asarray(logits_buffers[i][start:end])
  return lengths, out, out_logits


def resolve_parallelism_sizes(num_devices: int, tensor_parallel_size: int = -1, data_parallel_size: int = -1,
                              expert_parallel_size: int = 1) -> Tuple[int, int, int]:
  """Fills -1 entries so that tp * dp == num_devices (ep reuses the same ranks)."""
  tp, dp, ep = tensor_parallel_size, data_parallel_size, expert_parallel_size
  if tp <= 0 and dp <= 0:
    tp, dp = num_devices, 1
  elif tp <= 0:
    if num_devices % dp:
      raise ValueError(f"data_parallel_size {dp} does not divide {num_devices} devices")
    tp = num_devices // dp
  elif dp <= 0:
    if num_devices % tp:
      raise ValueError(f"tensor_parallel_size {tp} does not divide {num_devices} devices")
    dp = num_devices // tp
  if tp * dp != num_devices:
    raise ValueError(f"tensor_parallel_size * data_parallel_size = {tp * dp} != {num_devices} devices")
  return tp, dp, max(1, ep)


# ---- weight transfer ---------------------------------------------------------------------------
def build_flat_dict(flat_state: Iterable[Tuple[str, torch.Tensor]],
                    mappings: Mapping[str, Tuple[str, Any]]) -> Dict[str, Tuple[torch.Tensor, Any]]:
  """Resolves destination keys against a mapping `{source pattern: (dst pattern, spec)}` where `*`
  stands for a layer index. Returns `{source key: (dst tensor, spec)}`. Destination keys that
  no pattern produces are an error, as are patterns matching nothing."""
  dst = dict(flat_state)
  out: Dict[str, Tuple[torch.Tensor, Any]] = {}
  used = set()
  for src_pat, (dst_pat, spec) in mappings.items():
    if "*" not in dst_pat:
      if dst_pat in dst:
        out[src_pat] = (dst[dst_pat], spec)
        used.add(dst_pat)
      continue
    rx = re.compile("^" + re.escape(dst_pat).replace(r"\*", r"(\d+)") + "$")
    for k, v in dst.items():
      m = rx.match(k)
      if m:
        src_key = src_pat
        for g in m.groups():
          src_key = src_key.replace("*", g, 1)
        out[src_key] = (v, spec)
        used.add(k)
  missing = set(dst) - used
  if missing:
    raise KeyError(f"no mapping produces destination keys: {sorted(missing)[:8]}")
  return out


def _align_shape(src: torch.Tensor, dst_shape: Sequence[int], key: str) -> torch.Tensor:
  """Repeats (KV-head replication) or zero-pads (head-dim padding) `src` to reach `dst_shape`."""
  if tuple(src.shape) == tuple(dst_shape):
    return src
  if src.dim() != len(dst_shape):
    raise ValueError(f"rank mismatch for {key}: {tuple(src.shape)} vs {tuple(dst_shape)}")
  out = src
  for ax, (s, d) in enumerate(zip(src.shape, dst_shape)):
    if s == d:
      continue
    if d % s == 0 and ("k_proj" in key or "v_proj" in key or "kv" in key) and d > s and d // s <= 64 and ax != out.dim() - 1:
      out = out.repeat_interleave(d // s, dim=ax)
    elif d > s:
      pad = [0, 0] * out.dim()
      pad[2 * (out.dim() - 1 - ax) + 1] = d - s
      out = torch.nn.functional.pad(out, pad)
    else:
      raise ValueError(f"cannot align {key}: {tuple(src.shape)} -> {tuple(dst_shape)}")
  return out


@torch.no_grad()
def transfer_state_with_mappings(src_state: Mapping[str, torch.Tensor], dst_state: Mapping[str, torch.Tensor],
                                 key_mappings: Mapping[str, Tuple[str, Any]],
                                 key_mapping_hook_fns: Optional[Mapping[str, Callable]] = None,
                                 transpose_keys: Optional[Mapping[str, Tuple[int, ...]]] = None,
                                 reshard_fn: Optional[Callable] = None, tie_lm_head: Optional[Tuple[str, str]] = None,
                                 **_unused) -> Mapping[str, torch.Tensor]:
  """Copies `src_state` into `dst_state` (in place) through a key mapping: optional transpose per
  key suffix, optional hook function, shape alignment by repeat / zero-pad, dtype cast, and a
  tied lm_head (`(embedding key, lm_head key)`) kept in sync."""
  pairs = build_flat_dict(dst_state.items(), key_mappings)
  for src_key, (dst_t, spec) in pairs.items():
    if src_key not in src_state:
      raise KeyError(f"source state has no key {src_key}")
    v = src_state[src_key]
    for suffix, perm in (transpose_keys or {}).items():
      if src_key.endswith(suffix):
        v = v.permute(*perm)
    for pat, fn in (key_mapping_hook_fns or {}).items():
      if re.search(pat, src_key):
        v = fn(v)
    v = _align_shape(v, dst_t.shape, src_key)
    if reshard_fn is not None:
      v = reshard_fn(v, spec)
    dst_t.copy_(v.to(dst_t.dtype))
  if tie_lm_head is not None:
    emb, head = tie_lm_head
    if emb in dst_state and head in dst_state:
      dst_state[head].copy_(dst_state[emb].t() if dst_state[head].shape != dst_state[emb].shape else dst_state[emb])
  return dst_state


# ---- direct (same naming family) transfer -------------------------------------------------------
_LAYER_INDEX = re.compile(r"(^|\.)(layers)\.(\d+)\.")
_WRAPPERS_SRC = ("base",)          # a trainer state that wraps the parameters once
_WRAPPERS_DST = ("model",)         # serving wrappers nest the model, possibly several times


def flatten_state(tree: Mapping[str, Any], prefix: str = "") -> Dict[str, torch.Tensor]:
  """Nested mappings of tensors -> {dotted key: tensor}. Already flat states pass through."""
  flat: Dict[str, torch.Tensor] = {}
  for k, v in tree.items():
    key = f"{prefix}{k}"
    if isinstance(v, Mapping):
      flat.update(flatten_state(v, key + "."))
    else:
      flat[key] = v
  return flat


def _unwrap(tree: Mapping[str, Any], wrappers: Sequence[str], repeatedly: bool) -> Mapping[str, Any]:
  while isinstance(tree, Mapping) and len(tree) >= 1:
    hit = next((w for w in wrappers if w in tree and isinstance(tree[w], Mapping)), None)
    if hit is None:
      break
    tree = tree[hit]
    if not repeatedly:
      break
  return tree


def stacked_key(per_layer_key: str) -> Optional[Tuple[str, int]]:
  """`a.layers.7.b` -> (`a.layers.b`, 7): the key under which a layer-stacked ("scanned") state keeps the same
  parameter, and the layer's index. None for keys outside the layer stack."""
  m = _LAYER_INDEX.search(per_layer_key)
  if m is None:
    return None
  return per_layer_key[:m.start(3)] + per_layer_key[m.end(3) + 1:], int(m.group(3))


def unstack_scanned(stacked: torch.Tensor, layer: int, scan_axis: int) -> torch.Tensor:
  """Layer `layer` of a parameter stacked along `scan_axis` (a view, no copy)."""
  return stacked.select(scan_axis, layer)


def fuse_moe_gate_up(gate: torch.Tensor, up: torch.Tensor, interleave: bool = False) -> torch.Tensor:
  """Separate expert gate (`wi_0`) and up (`wi_1`) projections [..., F, D] -> one fused [..., 2 F, D] weight:
  gate rows then up rows (the layout of this package's `gate_up_proj`), or row-interleaved g0,u0,g1,u1,... for
  engines that want the pair adjacent."""
  if gate.shape != up.shape:
    raise ValueError(f"gate {tuple(gate.shape)} and up {tuple(up.shape)} projections differ in shape")
  if not interleave:
    return torch.cat((gate, up), dim=-2)
  return torch.stack((gate, up), dim=-2).reshape(*gate.shape[:-2], 2 * gate.shape[-2], gate.shape[-1])


def _lookup(key: str, rank: int, src: Mapping[str, torch.Tensor], scan_axis: int) -> Optional[torch.Tensor]:
  """`key` in the source, or its layer's slice of a stacked source parameter of rank `rank + 1`."""
  if key in src:
    return src[key]
  where = stacked_key(key)
  if where is not None and where[0] in src:
    stacked, layer = src[where[0]], where[1]
    if stacked.dim() == rank + 1 and layer < stacked.shape[scan_axis]:
      return unstack_scanned(stacked, layer, scan_axis)
  return None


_FUSED_FROM = (("gate_up_proj", ("gate_proj", "up_proj")), ("wi", ("wi_0", "wi_1")))


def _source_for(key: str, dst_t: torch.Tensor, src: Mapping[str, torch.Tensor], scan_axis: int
                ) -> Optional[torch.Tensor]:
  """The source tensor that fills destination `key`: the same key (or the layer's slice where the source keeps
  layers stacked); or, when the destination wants gate|up fused and the source has them apart, the fusion."""
  found = _lookup(key, dst_t.dim(), src, scan_axis)
  if found is not None:
    return found
  for fused, (gate_name, up_name) in _FUSED_FROM:
    if fused in key:
      gate = _lookup(key.replace(fused, gate_name), dst_t.dim(), src, scan_axis)
      up = _lookup(key.replace(fused, up_name), dst_t.dim(), src, scan_axis)
      if gate is not None and up is not None:
        return fuse_moe_gate_up(gate, up)
  return None


def _stack_into(dst_t: torch.Tensor, key: str, src: Mapping[str, torch.Tensor], scan_axis: int) -> bool:
  """Fills a layer-stacked destination from per-layer source keys. True if every layer was found."""
  marker = ".layers."
  if marker not in key and not key.startswith("layers."):
    return False
  head, _, tail = key.partition("layers.")
  n = dst_t.shape[scan_axis]
  parts = [src.get(f"{head}layers.{i}.{tail}") for i in range(n)]
  if any(p is None for p in parts):
    return False
  for i, part in enumerate(parts):
    dst_t.select(scan_axis, i).copy_(_align_shape(part, dst_t.select(scan_axis, i).shape, key).to(dst_t.dtype))
  return True


@torch.no_grad()
def transfer_state_directly(src_state: Mapping[str, Any], dst_state: Mapping[str, Any],
                            reshard_fn: Optional[Callable] = None, scan_axis: int = 0,
                            delete_dst_buffers: bool = False, reshard_chunk_size: Optional[int] = None
                            ) -> Mapping[str, Any]:
  """Copies a state into another one of the same naming family by structure, without a key mapping.

  * wrappers are stripped: one `base` level on the source (a trainer state), any depth of `model` on the
    destination (serving wrappers); nested mappings are matched by dotted key;
  * keys only one side has (KV caches, RNG state) are skipped; no common key at all is an error;
  * layer stacks: if one side keeps a parameter stacked over layers (`layers.w`, [L, ...] along `scan_axis`) and
    the other per layer (`layers.3.w`), slices are taken or filled accordingly;
  * separate expert gate / up projections on the source are fused for a destination that holds `gate_up_proj`;
  * `reshard_chunk_size` bounds how many keys are in flight at once: the copies of a chunk are issued, then the
    stream is drained before the next chunk, so temporaries (casts, fused or re-laid-out tensors) of at most one
    chunk are alive at a time;
  * `delete_dst_buffers` frees each destination tensor's storage right before it is re-created from the source
    (not when the two alias), which lowers the peak when source and destination share a GPU.
  """
  src = flatten_state(_unwrap(src_state, _WRAPPERS_SRC, repeatedly=False))
  dst = flatten_state(_unwrap(dst_state, _WRAPPERS_DST, repeatedly=True))
  keys = list(dst)
  step = max(1, reshard_chunk_size or len(keys) or 1)
  moved = 0
  for start in range(0, len(keys), step):
    for key in keys[start:start + step]:
      dst_t = dst[key]
      value = _source_for(key, dst_t, src, scan_axis)
      if value is None:
        moved += int(_stack_into(dst_t, key, src, scan_axis))
        continue
      if reshard_fn is not None:
        value = reshard_fn(value, None)
      value = _align_shape(value, dst_t.shape, key)
      if delete_dst_buffers and value.data_ptr() != dst_t.data_ptr():
        shape, dtype, device = dst_t.shape, dst_t.dtype, dst_t.device
        dst_t.data = torch.empty(0, dtype=dtype, device=device)              # release before re-creating
        dst_t.data = value.to(device=device, dtype=dtype, copy=True).reshape(shape)
      else:
        dst_t.copy_(value.to(dst_t.dtype))
      moved += 1
    if reshard_chunk_size and torch.cuda.is_available() and any(t.is_cuda for t in dst.values()):
      torch.cuda.synchronize()
  if moved == 0:
    raise ValueError("source and destination states share no keys")
  return dst_state


def verify_state_closeness(a: Mapping[str, torch.Tensor], b: Mapping[str, torch.Tensor], atol: float = 1e-2) -> bool:
  if set(a) != set(b):
    return False
  return all(torch.allclose(a[k].float().cpu(), b[k].float().cpu(), atol=atol) for k in a)
