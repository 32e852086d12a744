"""Named meshes over ranks.

The reference describes parallelism with `jax.sharding.Mesh(devices, axis_names)` inside one
controller process (tunix/utils/mesh.py:51). Here every GPU has its own process; a `Mesh` is an
n-dimensional array of global ranks with axis names ("fsdp", "tp", "dp", "ep", "sp"), and each
axis maps to a `torch.distributed` process group made of the ranks that differ only along that
axis. A role of an RL cluster (actor, rollout, ...) gets its own mesh over a subset of ranks.
"""
from __future__ import annotations

import itertools
import os
import threading
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.distributed as dist

_CURRENT: Optional["Mesh"] = None
_GROUP_CACHE: Dict[Tuple[int, ...], object] = {}
_LOCK = threading.Lock()

DATA_AXES = ("dp", "fsdp", "data")


def world_size() -> int:
  return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def rank() -> int:
  return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def local_rank() -> int:
  return int(os.environ.get("LOCAL_RANK", "0"))


def default_device() -> Optional[torch.device]:
  if _CURRENT is not None:
    return _CURRENT.device
  return None


def init_distributed(backend: Optional[str] = None, timeout_s: float = 1800.0) -> None:
  """Initialises `torch.distributed` from the torchrun environment (no-op when already
  initialised or when WORLD_SIZE is 1/unset). NCCL on GPUs, gloo on CPU."""
  import datetime
  if dist.is_initialized() or int(os.environ.get("WORLD_SIZE", "1")) <= 1:
    return
  if backend is None:
    backend = "nccl" if torch.cuda.is_available() else "gloo"
  if backend == "nccl":
    torch.cuda.set_device(local_rank())
  os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
  kw = {}
  if backend == "nccl":
    kw["device_id"] = torch.device("cuda", local_rank())
  dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)


def _group_for(ranks: Tuple[int, ...]):
  """Process group over `ranks` (cached). Must be called collectively by all ranks in the
  same order, which `Mesh.__init__` guarantees by enumerating every group of every axis."""
  if not dist.is_initialized() or len(ranks) <= 1:
    return None
  with _LOCK:
    g = _GROUP_CACHE.get(ranks)
    if g is None:
      g = dist.new_group(list(ranks))
      _GROUP_CACHE[ranks] = g
    return g


class Mesh:
  """An array of global ranks with named axes.

  `Mesh((4, 2), ("fsdp", "tp"))` over 8 ranks puts ranks 0..7 in row-major order; rank r then
  has a coordinate per axis, `group(axis)` is the process group along that axis and
  `axis_size(axis)` its size. `ranks` may select any subset/ordering of the world.
  """

  def __init__(self, shape: Sequence[int], axis_names: Sequence[str], ranks: Optional[Sequence[int]] = None,
               build_groups: bool = True):
    shape = tuple(int(s) for s in shape)
    n = int(np.prod(shape)) if shape else 1
    if ranks is None:
      ranks = list(range(n))
    ranks = list(ranks)
    if len(ranks) != n:
      raise ValueError(f"mesh shape {shape} needs {n} ranks, got {len(ranks)}")
    if len(shape) != len(axis_names):
      raise ValueError("shape and axis_names must have the same length")
    self.shape = shape
    self.axis_names = tuple(axis_names)
    self.devices = np.array(ranks, dtype=np.int64).reshape(shape)
    self._groups: Dict[str, object] = {}
    self._all_group = None
    me = rank()
    self.contains_me = me in ranks
    if build_groups and dist.is_available() and dist.is_initialized():
      # every rank of the world walks the same list of groups in the same order
      for ax_i, ax in enumerate(self.axis_names):
        other = [range(s) for i, s in enumerate(shape) if i != ax_i]
        for combo in itertools.product(*other):
          idx = list(combo)
          idx.insert(ax_i, slice(None))
          members = tuple(int(r) for r in self.devices[tuple(idx)])
          g = _group_for(members)
          if me in members:
            self._groups[ax] = g
      self._all_group = _group_for(tuple(sorted(int(r) for r in ranks))) if n > 1 else None

  # ---- queries ---------------------------------------------------------------------
  @property
  def size(self) -> int:
    return int(self.devices.size)

  @property
  def empty(self) -> bool:
    return self.devices.size == 0

  @property
  def device(self) -> Optional[torch.device]:
    if torch.cuda.is_available():
      return torch.device("cuda", local_rank())
    return torch.device("cpu")

  def axis_size(self, axis: str) -> int:
    if axis not in self.axis_names:
      return 1
    return self.shape[self.axis_names.index(axis)]

  def coords(self, r: Optional[int] = None) -> Dict[str, int]:
    r = rank() if r is None else r
    pos = np.argwhere(self.devices == r)
    if len(pos) == 0:
      raise ValueError(f"rank {r} is not part of mesh {self}")
    return {ax: int(pos[0][i]) for i, ax in enumerate(self.axis_names)}

  def axis_index(self, axis: str) -> int:
    if axis not in self.axis_names or not self.contains_me:
      return 0
    return self.coords()[axis]

  def group(self, axis: str):
    """Process group of the ranks that share all coordinates but `axis` with this rank."""
    return self._groups.get(axis)

  def all_group(self):
    return self._all_group

  def data_coords(self, axes: Sequence[str]) -> Tuple[int, int]:
    """(index, size) of this rank in the flattened product of the given data axes."""
    idx, size = 0, 1
    if not self.contains_me:
      return 0, 1
    c = self.coords()
    for ax in self.axis_names:
      if ax in axes:
        idx = idx * self.axis_size(ax) + c[ax]
        size *= self.axis_size(ax)
    return idx, size

  def ranks(self) -> List[int]:
    return [int(r) for r in self.devices.reshape(-1)]

  def __eq__(self, other):
    return (isinstance(other, Mesh) and self.shape == other.shape and self.axis_names == other.axis_names
            and np.array_equal(self.devices, other.devices))

  def __hash__(self):
    return hash((self.shape, self.axis_names, tuple(self.ranks())))

  def __repr__(self):
    return f"Mesh(shape={self.shape}, axis_names={self.axis_names}, ranks={self.ranks()})"

  def __enter__(self):
    self._prev = current_mesh()
    set_current_mesh(self)
    return self

  def __exit__(self, *exc):
    set_current_mesh(self._prev)
    return False


def create_mesh(shape: Sequence[int], axis_names: Sequence[str], ranks: Optional[Sequence[int]] = None) -> Mesh:
  """Counterpart of `tunix.utils.mesh.create_mesh`: a mesh over the first prod(shape) ranks
  (or the given ones). On an NVSwitch box every GPU pair has the same bandwidth, so there is
  no topology-dependent placement to do."""
  return Mesh(shape, axis_names, ranks)


def current_mesh() -> Optional[Mesh]:
  return _CURRENT


def set_current_mesh(m: Optional[Mesh]) -> None:
  global _CURRENT
  _CURRENT = m
