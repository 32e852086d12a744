"""Moving parameter trees between role layouts (tunix/rl/reshard.py:33-280).

The reference re-shards with a cross-mesh `device_put`. Here a parameter tree is a `{name: tensor}` dict and
there are three cases, picked per leaf by comparing source and target:

  * same storage: passed through;
  * same shape: one device copy with a dtype cast (trainer and rollout replica on one GPU, or a host-offloaded
    tree coming back);
  * the target is a tensor-parallel slice of the source (`tp`, `tp_rank` and the model config are given): the
    2-D blocks that make up the slice come from `dist.weight_sync.tp_blocks` - the same block table the
    one-launch transfer kernel walks - and are copied block by block. This is the fallback for trees that do
    not live in a flat parameter buffer.

Trainer ranks whose parameters live in a `FlatParamStore` do not come through here: `dist.weight_sync.
RolloutReplica.sync()` moves the whole model with one kernel launch that reads a trainer rank's buffer through
its peer mapping (see `rl/rollout/native_rollout.py::update_params`).
"""
from __future__ import annotations

import logging
import time
from typing import Any, Dict, Mapping, Optional

import torch

log = logging.getLogger(__name__)


def _copy_blocks(src: torch.Tensor, dst: torch.Tensor, blocks) -> None:
  """Fills `dst` from 2-D blocks (source row, source col, rows, cols, destination row) of `src`."""
  s2 = src.reshape(src.shape[0], -1) if src.dim() > 1 else src.reshape(1, -1)
  d2 = dst.reshape(dst.shape[0], -1) if dst.dim() > 1 else dst.reshape(1, -1)
  for (r0, c0, nr, nc, dr) in blocks:
    if src.dim() > 1:
      d2[dr:dr + nr, :nc].copy_(s2[r0:r0 + nr, c0:c0 + nc], non_blocking=True)
    else:                                   # vectors: `dr` is the destination column
      d2[0, dr:dr + nc].copy_(s2[0, c0:c0 + nc], non_blocking=True)


@torch.no_grad()
def reshard_pytree(source: Mapping[str, torch.Tensor], target: Mapping[str, torch.Tensor], cache_plan: bool = True,
                   donate_input: bool = False, use_experimental_pre_reshard: bool = True, *, model_config: Any = None,
                   tp: int = 1, tp_rank: int = 0, shard_vocab: bool = False) -> Dict[str, torch.Tensor]:
  """Returns `source` laid out like `target` (device, dtype and shape of every leaf).

  `cache_plan` and `use_experimental_pre_reshard` tune the reference's cross-mesh transfer and have no
  counterpart here (block tables are cheap to rebuild). With `donate_input` the source leaves that were copied
  release their storage."""
  del cache_plan, use_experimental_pre_reshard
  t0 = time.time()
  out: Dict[str, torch.Tensor] = {}
  for name, dst in target.items():
    if name not in source:
      raise KeyError(f"source tree has no leaf {name}")
    src = source[name]
    if src.data_ptr() == dst.data_ptr() and src.shape == dst.shape:
      out[name] = src
      continue
    if tuple(src.shape) == tuple(dst.shape):
      out[name] = src.to(device=dst.device, dtype=dst.dtype, non_blocking=True)
    else:
      if tp <= 1 or model_config is None:
        raise ValueError(f"shape mismatch for {name}: {tuple(src.shape)} vs {tuple(dst.shape)} "
                         "(pass model_config, tp and tp_rank if the target is a tensor-parallel slice)")
      from ..dist import weight_sync
      shape, blocks = weight_sync.tp_blocks(name, src.shape, model_config, tp, tp_rank, shard_vocab)
      if tuple(shape) != tuple(dst.shape):
        raise ValueError(f"{name}: rank {tp_rank}/{tp} slice of {tuple(src.shape)} is {tuple(shape)}, "
                         f"target has {tuple(dst.shape)}")
      fresh = torch.empty(shape, dtype=dst.dtype, device=dst.device)
      _copy_blocks(src.to(device=dst.device, dtype=dst.dtype, non_blocking=True) if src.device != dst.device else
                   src.to(dst.dtype), fresh, blocks)
      out[name] = fresh
    if donate_input and out[name] is not src:
      src.data = torch.empty(0, dtype=src.dtype, device=src.device)
  log.debug("reshard_pytree: %d leaves in %.3f s", len(out), time.time() - t0)
  return out


def reshard_model_to_mesh(model: torch.nn.Module, mesh: Any) -> torch.nn.Module:
  """Places a model according to a role mesh: on this rank's GPU when the rank is part of the mesh; FSDP / TP
  sharding is then applied by `tunix_b200.dist`."""
  if mesh is None or not getattr(mesh, "contains_me", True):
    return model
  dev = mesh.device
  if dev is not None and next(model.parameters()).device != dev:
    model.to(dev)
  return model
