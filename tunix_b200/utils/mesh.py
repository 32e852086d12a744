"""Carving one pool of GPUs into the meshes of the RL roles (role of tunix/utils/mesh.py:
topology-aware sub-mesh allocation with COMPACT and PERFORMANCE policies).

`allocate_named_mesh_device_slices([(name, size), ...], devices, policy)` hands every request a
disjoint set of ranks:
  COMPACT      first-fit on the lowest free ranks, largest request first - wastes nothing, may
               straddle a socket or node boundary;
  PERFORMANCE  each request starts on the boundary of the smallest natural unit that holds it
               (power-of-two group inside a socket, whole node, whole nodes), so a slice never
               straddles a boundary it could have avoided; may leave holes.
A request that cannot be met raises with the free map in the message. `create_mesh` builds the
named `dist.mesh.Mesh` over an allocated slice.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

from ..dist import mesh as dist_mesh
from . import topology

COMPACT, PERFORMANCE = "COMPACT", "PERFORMANCE"
Mesh = dist_mesh.Mesh


def normalize_allocation_policy(policy: Optional[str]) -> str:
  if policy is None or policy == "":
    return COMPACT
  p = str(policy).strip().upper()
  if p not in (COMPACT, PERFORMANCE):
    raise ValueError(f"Unsupported mesh allocation policy {policy!r}; expected one of {COMPACT}, {PERFORMANCE}.")
  return p


def _free_runs(free: List[bool]) -> List[Tuple[int, int]]:
  runs, i = [], 0
  while i < len(free):
    if free[i]:
      j = i
      while j < len(free) and free[j]:
        j += 1
      runs.append((i, j - i))
      i = j
    else:
      i += 1
  return runs


def allocate_named_mesh_device_slices(requirements: Sequence[Tuple[str, int]], devices: Sequence[int],
                                      allocation_policy: str = COMPACT,
                                      topo: topology.NodeTopology = topology.HGX_B200) -> Dict[str, List[int]]:
  policy = normalize_allocation_policy(allocation_policy)
  devices = list(devices)
  total = sum(n for _, n in requirements)
  if total > len(devices):
    raise ValueError(f"mesh requests need {total} devices but only {len(devices)} are available: {list(requirements)}")
  names = [n for n, _ in requirements]
  if len(set(names)) != len(names):
    raise ValueError(f"duplicate mesh names in {names}")
  free = [True] * len(devices)
  out: Dict[str, List[int]] = {}
  order = sorted(range(len(requirements)), key=lambda i: -requirements[i][1])   # largest first, stable
  for i in order:
    name, size = requirements[i]
    if size <= 0:
      raise ValueError(f"mesh {name!r} asks for {size} devices")
    start = None
    if policy == PERFORMANCE:
      block = topo.aligned_block(size)
      for s in range(0, len(devices) - size + 1, block):
        if all(free[s:s + size]):
          start = s
          break
    if start is None and policy == COMPACT:
      # best fit: the smallest free run that holds the request
      fits = [(length, s) for s, length in _free_runs(free) if length >= size]
      if fits:
        start = min(fits)[1]
    if start is None:
      raise ValueError(f"cannot place mesh {name!r} of {size} devices under policy {policy}; free map: "
                       f"{''.join('.' if f else 'x' for f in free)}")
    for k in range(start, start + size):
      free[k] = False
    out[name] = devices[start:start + size]
  return out


def create_mesh(axis_shapes: Sequence[int], axis_names: Sequence[str], devices: Optional[Sequence[int]] = None) -> Mesh:
  n = 1
  for s in axis_shapes:
    n *= int(s)
  if devices is not None and len(devices) != n:
    raise ValueError(f"mesh shape {tuple(axis_shapes)} needs {n} devices, got {len(devices)}")
  return dist_mesh.create_mesh(axis_shapes, axis_names, ranks=list(devices) if devices is not None else None)


def describe(slices: Dict[str, List[int]], topo: topology.NodeTopology = topology.HGX_B200) -> Dict[str, Dict[str, int]]:
  out = {}
  for name, ranks in slices.items():
    nodes, sockets = topology.crossings(ranks, topo)
    out[name] = {"size": len(ranks), "nodes": nodes, "sockets": sockets}
  return out
