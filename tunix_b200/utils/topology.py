"""Node topology that the mesh allocator reasons about (role of tunix/utils/topology.py, which
lists TPU slice shapes).

An HGX B200 node: 8 GPUs, every pair connected at full NVLink 5 bandwidth through NVSwitch, so
inside a node every subset of GPUs is equally well connected; what distinguishes subsets is
the host side - two CPU sockets with four GPUs each (PCIe / NIC / NUMA locality) - and, across
nodes, the node boundary itself (NVLink inside, InfiniBand between). A topology is therefore a
tree: cluster -> nodes -> sockets -> GPUs, described by `(gpus_per_socket, sockets_per_node)`.
"""
from __future__ import annotations

import dataclasses
from typing import List, Sequence, Tuple


@dataclasses.dataclass(frozen=True)
class NodeTopology:
  gpus_per_socket: int = 4
  sockets_per_node: int = 2

  @property
  def gpus_per_node(self) -> int:
    return self.gpus_per_socket * self.sockets_per_node

  def node_of(self, rank: int) -> int:
    return rank // self.gpus_per_node

  def socket_of(self, rank: int) -> int:
    return rank // self.gpus_per_socket

  def aligned_block(self, size: int) -> int:
    """Smallest natural unit (socket, node, multiple of nodes) that holds `size` GPUs."""
    if size <= self.gpus_per_socket:
      b = 1
      while b < size:
        b *= 2
      return b
    if size <= self.gpus_per_node:
      return self.gpus_per_node
    n = self.gpus_per_node
    return ((size + n - 1) // n) * n


HGX_B200 = NodeTopology(4, 2)
SUPPORTED_SLICE_SIZES: Tuple[int, ...] = (1, 2, 4, 8)     # per node; multiples of 8 across nodes


def is_supported_slice(size: int, topo: NodeTopology = HGX_B200) -> bool:
  return size in SUPPORTED_SLICE_SIZES or (size > topo.gpus_per_node and size % topo.gpus_per_node == 0)


def crossings(ranks: Sequence[int], topo: NodeTopology = HGX_B200) -> Tuple[int, int]:
  """(number of distinct nodes, number of distinct sockets) a set of ranks touches."""
  return len({topo.node_of(r) for r in ranks}), len({topo.socket_of(r) for r in ranks})
