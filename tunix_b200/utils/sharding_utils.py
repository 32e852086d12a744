"""Placing a tensor according to a named-axis spec (tunix/utils/sharding_utils.py:24-45).

`shard(x, ("fsdp", None))` under a current mesh returns this rank's block of `x`: dimension d is cut
into `mesh.axis_size(spec[d])` equal parts and the part at the rank's coordinate is kept. The reference
leaves the data movement to the compiler (`with_sharding_constraint`); here the caller holds the full
value (every rank computed or loaded it) and takes its slice - the `eager` flag is accepted for API
parity and makes the slice a contiguous copy instead of a view. Without a mesh, or on CPU, `x` is
returned unchanged, as in the reference."""
from __future__ import annotations

from typing import Optional, Sequence, Union

import torch

Axis = Optional[Union[str, Sequence[str]]]


def shard(x: torch.Tensor, s: Sequence[Axis], eager: bool = False) -> torch.Tensor:
  from ..dist import mesh as mesh_lib
  mesh = mesh_lib.current_mesh()
  x = torch.as_tensor(x)
  if mesh is None or mesh.empty or not mesh.contains_me or not x.is_cuda:
    return x
  if len(s) > x.dim():
    raise ValueError(f"spec {tuple(s)} has more entries than the tensor has dimensions ({x.dim()})")
  out = x
  for d, axes in enumerate(s):
    if axes is None:
      continue
    names = (axes,) if isinstance(axes, str) else tuple(axes)
    index, parts = mesh.data_coords(names) if len(names) > 1 else (mesh.axis_index(names[0]), mesh.axis_size(names[0]))
    if parts == 1:
      continue
    if out.shape[d] % parts:
      raise ValueError(f"dimension {d} of size {out.shape[d]} does not divide over {parts} ranks of {names}")
    step = out.shape[d] // parts
    out = out.narrow(d, index * step, step)
  return out.contiguous() if eager else out
