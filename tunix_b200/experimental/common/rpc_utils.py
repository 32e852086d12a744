"""What may cross a process boundary (tunix/experimental/common/rpc_utils.py).

Control-plane payloads are pickled and sent to other processes. A device tensor in such a payload is a
bug: pickling a CUDA tensor drags its storage through the host, and the receiver cannot assume the same
GPU (a peer-mapped pointer means nothing elsewhere). Bulk data goes over the data plane (peer-memory
copies, the weight-sync transport); what travels by RPC must be plain numpy / Python data.
"""
from __future__ import annotations

import dataclasses
from typing import Any

import numpy as np


def _describe(v: Any) -> str:
  t = type(v)
  return f"{t.__module__}.{t.__qualname__}"


def validate_wire_safe(obj: Any) -> None:
  """Raises TypeError at the first array-like value inside `obj` (nested dataclasses, dicts - keys too -,
  lists, tuples, sets) that is not a `numpy.ndarray`: torch tensors on any device, or any other object
  exposing `shape` and `dtype`. Cycles are tolerated."""
  seen = set()
  todo = [obj]
  while todo:
    v = todo.pop()
    if id(v) in seen:
      continue
    seen.add(id(v))
    if isinstance(v, (np.ndarray, np.generic, str, bytes, int, float, bool, type(None))):
      continue
    if dataclasses.is_dataclass(v) and not isinstance(v, type):
      todo.extend(getattr(v, f.name) for f in dataclasses.fields(v))
    elif isinstance(v, dict):
      todo.extend(v.keys())
      todo.extend(v.values())
    elif isinstance(v, (list, tuple, set, frozenset)):
      todo.extend(v)
    elif hasattr(v, "shape") and hasattr(v, "dtype"):
      raise TypeError(f"payload holds a {_describe(v)}; convert device arrays to numpy (`.detach().cpu().numpy()`) "
                      "before sending them over RPC")


def to_wire(obj: Any) -> Any:
  """Copy of `obj` with every torch tensor replaced by a numpy array (bf16 widened to fp32)."""
  import torch
  if isinstance(obj, torch.Tensor):
    t = obj.detach().cpu()
    return (t.float() if t.dtype == torch.bfloat16 else t).numpy()
  if dataclasses.is_dataclass(obj) and not isinstance(obj, type):
    return dataclasses.replace(obj, **{f.name: to_wire(getattr(obj, f.name)) for f in dataclasses.fields(obj)})
  if isinstance(obj, dict):
    return {k: to_wire(v) for k, v in obj.items()}
  if isinstance(obj, (list, tuple)):
    return type(obj)(to_wire(v) for v in obj)
  return obj
