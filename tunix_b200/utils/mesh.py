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


# ------------------------------------------------------------------------------------ stateful allocation
class DeviceAllocationState:
  """A pool of GPUs (any set of global ranks, holes allowed) from which role meshes are taken and given back
  while a job runs (tunix/utils/mesh.py:156-186, 1334-1705 keep such a state over TPU coordinates).

  The pool is seen through the node topology as a tree node -> socket -> GPU. A request of n GPUs is answered with
  the candidate set that, in this order,
    1. touches the fewest nodes (NVLink inside a node, the network between nodes),
    2. touches the fewest sockets (host-side locality),
    3. PERFORMANCE: starts on an aligned block and keeps whole units (a node-sized request takes a whole free node);
       COMPACT: leaves the least fragmentation behind (prefers to finish partially used sockets and nodes),
    4. has the lowest ranks (determinism).
  Requests larger than a node take whole free nodes first and the remainder from the best partial node. Every
  allocation is named; `release(name)` returns its GPUs to the pool."""

  def __init__(self, devices: Sequence[int], topo: topology.NodeTopology = topology.HGX_B200):
    if len(set(devices)) != len(devices):
      raise ValueError("duplicate ranks in the device pool")
    self.topo = topo
    self.free = sorted(int(d) for d in devices)
    self.taken: Dict[str, List[int]] = {}

  # ---- views
  def _by_unit(self, ranks: Sequence[int], unit) -> Dict[int, List[int]]:
    groups: Dict[int, List[int]] = {}
    for r in ranks:
      groups.setdefault(unit(r), []).append(r)
    return groups

  def summary(self) -> str:
    """One line per node: which GPUs are free ('.') and which allocation holds the others, for logs."""
    owner = {r: name for name, ranks in self.taken.items() for r in ranks}
    known = sorted(set(self.free) | set(owner))
    lines = []
    for node, ranks in sorted(self._by_unit(known, self.topo.node_of).items()):
      cells = ["." if r in self.free else owner[r][:1].upper() for r in ranks]
      lines.append(f"node {node}: " + "".join(cells) + f"  ({sum(c == '.' for c in cells)} free)")
    return "\n".join(lines)

  # ---- allocation
  def _pick_within_node(self, free_here: List[int], n: int, policy: str) -> Optional[List[int]]:
    if len(free_here) < n:
      return None
    sockets = self._by_unit(free_here, self.topo.socket_of)
    if policy == PERFORMANCE:
      block = self.topo.aligned_block(n)
      for start in range(min(free_here) // block * block, max(free_here) + 1, block):
        cand = [r for r in free_here if start <= r < start + block][:n]
        if len(cand) == n and len({self.topo.socket_of(r) for r in cand}) == max(1, -(-n // self.topo.gpus_per_socket)):
          return cand
    # fewest sockets; among those COMPACT finishes the fullest partially used socket first
    fits = [s for s in sockets.values() if len(s) >= n]
    if fits:
      best = min(fits, key=lambda s: (len(s) if policy == COMPACT else -len(s), s[0]))
      return best[:n]
    order = sorted(sockets.values(), key=lambda s: (-len(s), s[0]))
    flat = [r for s in order for r in s]
    return sorted(flat[:n])

  def allocate(self, name: str, n: int, policy: str = COMPACT) -> List[int]:
    policy = normalize_allocation_policy(policy)
    if name in self.taken:
      raise ValueError(f"allocation {name!r} already exists")
    if n <= 0:
      raise ValueError(f"mesh {name!r} asks for {n} devices")
    if n > len(self.free):
      raise ValueError(f"cannot place mesh {name!r} of {n} devices: {len(self.free)} free\n{self.summary()}")
    nodes = self._by_unit(self.free, self.topo.node_of)
    per_node = self.topo.gpus_per_node
    def one_node(pool: Dict[int, List[int]], want: int) -> List[int]:
      """`want` GPUs out of a single node of `pool` if one can hold them: the fullest-fitting node (COMPACT, keeps
      empty nodes whole) or the emptiest one (PERFORMANCE, keeps neighbours apart)."""
      holders = [(len(f), node) for node, f in pool.items() if len(f) >= want]
      if not holders:
        return []
      key = (lambda t: (t[0], t[1])) if policy == COMPACT else (lambda t: (-t[0], t[1]))
      return self._pick_within_node(pool[min(holders, key=key)[1]], want, policy) or []

    chosen: List[int] = one_node(nodes, n) if n <= per_node else []
    if not chosen:
      rest, pool = n, dict(nodes)
      for node in sorted(nd for nd, f in nodes.items() if len(f) == per_node):      # whole free nodes first
        if rest >= per_node:
          chosen += pool.pop(node)
          rest -= per_node
      if rest:
        tail = one_node(pool, rest)                                                  # the remainder from ONE node
        if not tail:                                                                 # ... or spread, fullest first
          for node in sorted(pool, key=lambda nd: (-len(pool[nd]), nd)):
            take = self._pick_within_node(pool[node], min(rest - len(tail), len(pool[node])), policy) or []
            tail += take
            if len(tail) == rest:
              break
        chosen += tail
        rest -= len(tail)
      if rest:
        raise ValueError(f"cannot place mesh {name!r} of {n} devices under policy {policy}\n{self.summary()}")
    chosen = sorted(chosen)
    self.free = [r for r in self.free if r not in set(chosen)]
    self.taken[name] = chosen
    return chosen

  def release(self, name: str) -> None:
    self.free = sorted(self.free + self.taken.pop(name))


def allocate_devices(requirements: Sequence[Tuple[str, int]], devices: Sequence[int], allocation_policy: str = COMPACT,
                     topo: topology.NodeTopology = topology.HGX_B200) -> Dict[str, List[int]]:
  """Named slices out of an arbitrary pool (holes, several nodes) through `DeviceAllocationState`; the largest
  request is placed first so that small ones fill the gaps."""
  state = DeviceAllocationState(devices, topo)
  for name, size in sorted(requirements, key=lambda r: -r[1]):
    state.allocate(name, size, allocation_policy)
  return {name: state.taken[name] for name, _ in requirements}
