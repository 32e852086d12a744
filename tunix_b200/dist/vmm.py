"""Peer-mapped device memory built directly on the CUDA virtual-memory-management driver calls.

`PeerHeap.alloc(nbytes)` gives every rank of a process group (one node, one process per GPU) a buffer on its own
GPU plus a device pointer to each peer's buffer, which this package's kernels read and write with plain loads and
stores over NVLink. Per allocation:

  1. `cuMemCreate`: physical memory on the local GPU, exportable as a POSIX file descriptor;
  2. `cuMemExportToShareableHandle`, then the descriptor travels to every local peer over abstract-namespace Unix
     sockets (`socket.send_fds`; the socket names derive from a token the group's rank 0 broadcasts);
  3. every rank imports the peers' descriptors (`cuMemImportFromShareableHandle`), reserves a virtual range per buffer
     (`cuMemAddressReserve`), maps it (`cuMemMap`) and grants its own device read-write access (`cuMemSetAccess`);
  4. the local buffer is handed to PyTorch as a tensor over the raw pointer (CUDA array interface), so it is usable
     as an ordinary tensor and never owned by the caching allocator.

Nothing here binds a multicast object: peers are reached by unicast mappings only, so a rank that leaves does not
disturb the other ranks' GPUs. Mappings live until `close()` (or process exit).
"""
from __future__ import annotations

import os
import socket
import uuid
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist


class VmmError(RuntimeError):
  pass


def _driver():
  from cuda.bindings import driver
  return driver


def _ok(result, what: str):
  """cuda-python returns (status, *values)."""
  status, *values = result if isinstance(result, tuple) else (result,)
  if int(status) != 0:
    raise VmmError(f"{what} failed with CUDA driver error {int(status)}")
  if not values:
    return None
  return values[0] if len(values) == 1 else tuple(values)


class _RawDeviceArray:
  """CUDA array interface over a raw device pointer (lets `torch.as_tensor` wrap it without a copy)."""

  def __init__(self, ptr: int, nbytes: int):
    self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3,
                                     "strides": None}


class PeerBuffer:
  """One symmetric allocation: `local` tensor (uint8 view; `.view(dtype)` it) and `ptrs[r]` for every rank."""

  def __init__(self, local: torch.Tensor, ptrs: List[int], nbytes: int):
    self.local, self.ptrs, self.nbytes = local, ptrs, nbytes


class PeerHeap:

  def __init__(self, group, device: torch.device):
    self.group = group if group is not None else dist.group.WORLD
    self.rank, self.world = dist.get_rank(self.group), dist.get_world_size(self.group)
    self.device = device
    self.cu = _driver()
    torch.cuda.set_device(device)
    torch.zeros(1, device=device)                       # makes sure the primary context exists and is current
    token = [uuid.uuid4().hex if self.rank == 0 else None]
    dist.broadcast_object_list(token, src=dist.get_global_rank(self.group, 0), group=self.group)
    self._token = token[0]
    self._serial = 0
    self._mappings: List[Tuple[int, int, object]] = []   # (virtual address, size, handle) to undo in close()
    self._keep: List[object] = []
    cu = self.cu
    prop = cu.CUmemAllocationProp()
    prop.type = cu.CUmemAllocationType.CU_MEM_ALLOCATION_TYPE_PINNED
    prop.location.type = cu.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
    prop.location.id = device.index if device.index is not None else torch.cuda.current_device()
    prop.requestedHandleTypes = cu.CUmemAllocationHandleType.CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR
    self._prop = prop
    self._granularity = int(_ok(cu.cuMemGetAllocationGranularity(
        prop, cu.CUmemAllocationGranularity_flags.CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity"))

  # ---- descriptor exchange over Unix sockets ---------------------------------------------------
  def _address(self, rank: int, serial: int) -> str:
    return f"\0tunix_b200_vmm_{self._token}_{serial}_{rank}"

  def _exchange(self, fd: int) -> Dict[int, int]:
    """Sends `fd` to every peer and returns {peer rank: received descriptor}."""
    serial = self._serial
    self._serial += 1
    listener = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    listener.bind(self._address(self.rank, serial))
    listener.listen(self.world)
    listener.settimeout(60.0)
    try:
      dist.barrier(group=self.group)                    # every listener exists before anybody connects
      for peer in range(self.world):
        if peer == self.rank:
          continue
        with socket.socket(socket.AF_UNIX, socket.SOCK_STREAM) as out:
          out.settimeout(60.0)
          out.connect(self._address(peer, serial))
          socket.send_fds(out, [self.rank.to_bytes(4, "little")], [fd])
      received: Dict[int, int] = {}
      while len(received) < self.world - 1:
        conn, _ = listener.accept()
        with conn:
          conn.settimeout(60.0)
          data, fds, _, _ = socket.recv_fds(conn, 4, 1)
          if len(data) != 4 or len(fds) != 1:
            raise VmmError("peer sent a malformed descriptor message")
          received[int.from_bytes(data, "little")] = fds[0]
      dist.barrier(group=self.group)
      return received
    finally:
      listener.close()

  # ---- mapping ---------------------------------------------------------------------------------
  def _map(self, handle, size: int) -> int:
    cu = self.cu
    va = int(_ok(cu.cuMemAddressReserve(size, self._granularity, 0, 0), "cuMemAddressReserve"))
    _ok(cu.cuMemMap(va, size, 0, handle, 0), "cuMemMap")
    access = cu.CUmemAccessDesc()
    access.location.type = cu.CUmemLocationType.CU_MEM_LOCATION_TYPE_DEVICE
    access.location.id = self._prop.location.id
    access.flags = cu.CUmemAccess_flags.CU_MEM_ACCESS_FLAGS_PROT_READWRITE
    _ok(cu.cuMemSetAccess(va, size, [access], 1), "cuMemSetAccess")
    self._mappings.append((va, size, handle))
    return va

  def alloc(self, nbytes: int) -> PeerBuffer:
    """Collective over the group: every rank calls it with the same size, in the same order."""
    cu = self.cu
    size = -(-int(nbytes) // self._granularity) * self._granularity
    handle = _ok(cu.cuMemCreate(size, self._prop, 0), "cuMemCreate")
    fd = int(_ok(cu.cuMemExportToShareableHandle(
        handle, cu.CUmemAllocationHandleType.CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle"))
    try:
      peer_fds = self._exchange(fd) if self.world > 1 else {}
    finally:
      os.close(fd)
    ptrs = [0] * self.world
    ptrs[self.rank] = self._map(handle, size)
    for peer, pfd in sorted(peer_fds.items()):
      try:
        imported = _ok(cu.cuMemImportFromShareableHandle(
            pfd, cu.CUmemAllocationHandleType.CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR), "cuMemImportFromShareableHandle")
      finally:
        os.close(pfd)
      ptrs[peer] = self._map(imported, size)
    raw = _RawDeviceArray(ptrs[self.rank], int(nbytes))
    local = torch.as_tensor(raw, device=self.device)
    self._keep.append(raw)
    local.zero_()
    return PeerBuffer(local, ptrs, int(nbytes))

  def close(self) -> None:
    cu = self.cu
    torch.cuda.synchronize(self.device)
    for va, size, handle in reversed(self._mappings):
      cu.cuMemUnmap(va, size)
      cu.cuMemAddressFree(va, size)
      cu.cuMemRelease(handle)
    self._mappings = []


def available() -> Optional[str]:
  """None when the driver bindings import and fd passing exists; else the reason."""
  try:
    _driver()
  except Exception as e:  # noqa: BLE001
    return f"cuda driver bindings do not import: {type(e).__name__}: {e}"
  if not hasattr(socket, "send_fds"):
    return "socket.send_fds is not available"
  return None
