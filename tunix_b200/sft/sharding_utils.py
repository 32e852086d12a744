"""Host -> device placement of input batches.

Every rank runs the same input pipeline; `shard_input` keeps this rank's slice of the leading
(batch) dimension for the data-parallel axes named in `data_sharding_axis` and moves it to the
rank's GPU through pinned memory. A batch that is not divisible by the data-parallel size is
replicated instead, as in tunix/sft/sharding_utils.py:25-95.
"""
from __future__ import annotations

import dataclasses
import logging
from typing import Any, Sequence, Tuple

import numpy as np
import torch

log = logging.getLogger(__name__)


def _dp_rank_size(axes: Sequence[str]) -> Tuple[int, int]:
  from ..dist import mesh as mesh_lib
  m = mesh_lib.current_mesh()
  if m is None:
    return 0, 1
  return m.data_coords(axes)


def _place(x: Any, rank: int, size: int, device) -> Any:
  if isinstance(x, np.ndarray):
    if x.dtype.kind in "OUS":
      return x
    x = torch.from_numpy(np.ascontiguousarray(x))
  if not isinstance(x, torch.Tensor):
    return x
  if size > 1 and x.dim() >= 1:
    if x.shape[0] % size == 0:
      per = x.shape[0] // size
      x = x[rank * per:(rank + 1) * per]
    else:
      log.warning("batch dim %d not divisible by data-parallel size %d; replicating", x.shape[0], size)
  if device is not None and x.device != device:
    if x.device.type == "cpu" and device.type == "cuda":
      x = x.contiguous().pin_memory().to(device, non_blocking=True)
    else:
      x = x.to(device)
  return x


def get_sharding(axes: Sequence[str] = ("fsdp",)):
  """(rank, size) of this process along the data-parallel axes."""
  return _dp_rank_size(axes)


def shard_input(batch: Any, data_sharding_axis: Sequence[str] = ("fsdp",), device=None) -> Any:
  """Applies `_place` to every array leaf of a dict / dataclass / tuple batch."""
  rank, size = _dp_rank_size(data_sharding_axis)
  if device is None:
    from ..dist import mesh as mesh_lib
    device = mesh_lib.default_device()

  def rec(x):
    if isinstance(x, dict):
      return {k: rec(v) for k, v in x.items()}
    if dataclasses.is_dataclass(x) and not isinstance(x, type):
      return dataclasses.replace(x, **{f.name: rec(getattr(x, f.name)) for f in dataclasses.fields(x)})
    if isinstance(x, (list, tuple)) and not isinstance(x, str):
      t = [rec(v) for v in x]
      return type(x)(t) if not hasattr(x, "_fields") else type(x)(*t)
    return _place(x, rank, size, device)

  return rec(batch)
