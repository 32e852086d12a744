"""Moving parameter trees between role layouts (tunix/rl/reshard.py:33-280).

The reference re-shards with a cross-mesh `device_put`. Here a parameter tree is a
`{name: tensor}` dict; within one process the copy is a device copy with a dtype cast, and
between ranks `tunix_b200.dist.weight_sync` pulls the needed slices straight out of the owner's
peer-mapped buffer."""
from __future__ import annotations

import logging
import threading
import time
from typing import Any, Dict, Mapping, Optional

import torch

log = logging.getLogger(__name__)


@torch.no_grad()
def reshard_pytree(source: Mapping[str, torch.Tensor], target: Mapping[str, torch.Tensor], cache_plan: bool = True,
                   donate_input: bool = False, use_experimental_pre_reshard: bool = True) -> Dict[str, torch.Tensor]:
  """Returns `source` laid out like `target` (device, dtype, shape of every leaf). Leaves that
  already alias the target storage are passed through."""
  del cache_plan, use_experimental_pre_reshard
  t0 = time.time()
  out: Dict[str, torch.Tensor] = {}
  for name, dst in target.items():
    if name not in source:
      raise KeyError(f"source tree has no leaf {name}")
    src = source[name]
    if tuple(src.shape) != tuple(dst.shape):
      raise ValueError(f"shape mismatch for {name}: {tuple(src.shape)} vs {tuple(dst.shape)}")
    if src.data_ptr() == dst.data_ptr():
      out[name] = src
    else:
      out[name] = src.to(device=dst.device, dtype=dst.dtype, non_blocking=True)
    if donate_input and out[name] is not src:
      src.data = torch.empty(0, dtype=src.dtype, device=src.device)
  log.debug("reshard_pytree: %d leaves in %.3f s", len(out), time.time() - t0)
  return out


def reshard_model_to_mesh(model: torch.nn.Module, mesh: Any) -> torch.nn.Module:
  """Places a model according to a role mesh: on this rank's GPU when the rank is part of the
  mesh; FSDP / TP sharding is then applied by `tunix_b200.dist`."""
  if mesh is None or not getattr(mesh, "contains_me", True):
    return model
  dev = mesh.device
  if dev is not None and next(model.parameters()).device != dev:
    model.to(dev)
  return model
