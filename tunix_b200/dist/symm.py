"""Symmetric (peer-mapped) buffers and the collectives built on them.

Two interchangeable backends provide the buffers, so that each process holds a device pointer to every peer's
copy (NVLink / NVSwitch peer access): `TUNIX_B200_SYMM_BACKEND=vmm` is this package's own allocator
(`dist/vmm.py`: `cuMemCreate` + descriptor passing over Unix sockets + `cuMemMap` of every peer's allocation);
`torch` delegates allocation and handle exchange to `torch.distributed._symmetric_memory` (a private torch API,
used for nothing else). The data movement itself is done by this package's own kernels
(`csrc/peer_comm.cu`), which read and write the peers' buffers with plain loads and stores from inside
the compute kernel:

  * `reduce_scatter_sum`  - pull-and-sum of the peers' fp32 gradient shards,
  * `adamw_allgather`     - AdamW on the local master shard, result pushed to every peer,
  * `barrier`             - flag exchange with a bounded spin; a timeout sets the status word
                            (`ops._lib.check_status` raises) instead of hanging the GPU.

No NVLS multicast object is bound here (plain peer loads/stores only), which keeps a rank that
exits early from disturbing its peers' GPUs.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib

_DEFAULT_BACKEND = "torch"       # "vmm": the own allocator of dist/vmm.py

_P, _I, _L, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _declare():
  lib = _lib.require()
  if getattr(lib, "_peer_declared", False):
    return lib
  lib.tx_peer_barrier.argtypes = [ctypes.POINTER(_P), _I, _I, _I, _L, _P, _P]
  lib.tx_peer_barrier.restype = _I
  lib.tx_reduce_scatter_grid.argtypes = []
  lib.tx_reduce_scatter_grid.restype = _I
  lib.tx_reduce_scatter_sum_f32.argtypes = [ctypes.POINTER(_P), _P, _L, _L, _I, _I, _P, _P]
  lib.tx_reduce_scatter_sum_f32.restype = _I
  lib.tx_reduce_scatter_sum_f32_bg.argtypes = [ctypes.POINTER(_P), _P, _L, _L, _I, _I, _I, _P]
  lib.tx_reduce_scatter_sum_f32_bg.restype = _I
  lib.tx_adamw_allgather.argtypes = [_P, _P, _P, _P, ctypes.POINTER(_P), _L, _L, _F, _F, _F, _F, _F, _F, _F, _P, _I, _I, _P]
  lib.tx_adamw_allgather.restype = _I
  lib.tx_peer_copy_2d.argtypes = [_P, _P, _L, _L, _L, _L, _P]
  lib.tx_peer_copy_2d.restype = _I
  lib._peer_declared = True
  return lib


def _ptr_array(ptrs: List[int]):
  arr = (_P * len(ptrs))()
  for i, p in enumerate(ptrs):
    arr[i] = p
  return arr


class SymmetricBuffers:
  """A set of named buffers allocated symmetrically on every rank of `group`."""

  def __init__(self, group, device: torch.device):
    from . import vmm
    backend = os.environ.get("TUNIX_B200_SYMM_BACKEND", _DEFAULT_BACKEND)
    if backend == "vmm" and vmm.available() is not None:
      raise RuntimeError(f"TUNIX_B200_SYMM_BACKEND=vmm: {vmm.available()}")
    self._heap = None
    self._sm = None
    self.group = group if group is not None else dist.group.WORLD
    if backend == "vmm":
      self._heap = vmm.PeerHeap(self.group, device)
    else:
      import torch.distributed._symmetric_memory as symm_mem
      self._sm = symm_mem
    self.world = dist.get_world_size(self.group)
    self.rank = dist.get_rank(self.group)
    self.device = device
    self.tensors: Dict[str, torch.Tensor] = {}
    self.handles: Dict[str, object] = {}
    self.peer_ptrs: Dict[str, List[int]] = {}
    self._epoch = 0
    self.wait_limit_ms = int(os.environ.get("TUNIX_PEER_WAIT_MS", "20000"))
    self.lib = _declare()
    # one int32 row of flags per rank (kMaxPeers = 16 entries)
    self.alloc("_flags", 16, torch.int32)
    self.alloc("_flags1", 16, torch.int32)      # second barrier channel: a side stream's barriers use their own flags
    self._epoch1 = 0

  def alloc(self, name: str, numel: int, dtype: torch.dtype) -> torch.Tensor:
    """Collective: every rank allocates the same buffers in the same order. Peer pointers are known at once with
    the own allocator, after `rendezvous()` with the torch backend; callers always rendezvous before use."""
    if self._heap is not None:
      itemsize = torch.empty((), dtype=dtype).element_size()
      buf = self._heap.alloc(numel * itemsize)
      t = buf.local.view(dtype)[:numel]
      self.tensors[name] = t
      self._pending_ptrs = getattr(self, "_pending_ptrs", {})
      self._pending_ptrs[name] = buf.ptrs
      return t
    t = self._sm.empty(numel, dtype=dtype, device=self.device)
    self.tensors[name] = t
    return t

  def rendezvous(self) -> None:
    """Collective: exchanges handles for every buffer allocated since the last call."""
    for name, t in self.tensors.items():
      if name in self.handles:
        continue
      if name in ("_flags", "_flags1"):
        t.zero_()
      if self._heap is not None:
        self.handles[name] = self._heap
        self.peer_ptrs[name] = [int(p) for p in self._pending_ptrs.pop(name)]
        continue
      h = self._sm.rendezvous(t, self.group)
      self.handles[name] = h
      self.peer_ptrs[name] = [int(p) for p in h.buffer_ptrs]
    torch.cuda.synchronize(self.device)
    dist.barrier(group=self.group)

  def ptrs_for(self, t: torch.Tensor) -> List[int]:
    """Peer pointers of a tensor that is (a view into) one of the symmetric buffers."""
    for name, base in self.tensors.items():
      lo = base.data_ptr()
      hi = lo + base.numel() * base.element_size()
      if lo <= t.data_ptr() < hi:
        off = t.data_ptr() - lo
        return [p + off for p in self.peer_ptrs[name]]
    raise ValueError("tensor is not part of a symmetric buffer")

  # ---- collectives ---------------------------------------------------------------------
  def barrier(self, channel: int = 0, stream=None) -> None:
    """Device-side barrier (bounded wait) on the current stream, or on `stream`. Barriers issued from two
    streams must use different channels: a channel is one flag row per rank plus its own epoch counter."""
    if channel == 0:
      self._epoch += 1
      epoch, name = self._epoch, "_flags"
    else:
      self._epoch1 += 1
      epoch, name = self._epoch1, "_flags1"
    sp = _lib.stream_ptr() if stream is None else stream.cuda_stream
    rc = self.lib.tx_peer_barrier(_ptr_array(self.peer_ptrs[name]), self.rank, self.world, epoch,
                                  self.wait_limit_ms, _lib.status_word(self.device).data_ptr(), sp)
    _lib.check_rc(rc, "tx_peer_barrier")

  def reduce_scatter_piece(self, full_fp32: torch.Tensor, out_piece: torch.Tensor, flat_start: int, stream=None,
                           background_ctas: int = 0) -> None:
    """out_piece = sum over ranks of full_fp32[flat_start : flat_start + n], read over NVLink. The caller has
    made sure (a barrier) that every rank's values in that range are final. With `background_ctas` the sum runs
    on that many long-lived CTAs, the form to use on a side stream while compute kernels own the machine."""
    sp = _lib.stream_ptr() if stream is None else stream.cuda_stream
    if background_ctas > 0:
      rc = self.lib.tx_reduce_scatter_sum_f32_bg(_ptr_array(self.ptrs_for(full_fp32)), out_piece.data_ptr(), flat_start,
                                                 out_piece.numel(), self.world, self.rank, background_ctas, sp)
      _lib.check_rc(rc, "tx_reduce_scatter_sum_f32_bg")
      return
    rc = self.lib.tx_reduce_scatter_sum_f32(_ptr_array(self.ptrs_for(full_fp32)), out_piece.data_ptr(), flat_start,
                                            out_piece.numel(), self.world, self.rank, None, sp)
    _lib.check_rc(rc, "tx_reduce_scatter_sum_f32")

  def reduce_scatter_sum(self, full_fp32: torch.Tensor, out_shard: torch.Tensor, rank: int) -> None:
    """out_shard = sum over ranks of full_fp32[rank * n : (rank + 1) * n], read over NVLink."""
    self.barrier()      # every rank's gradients are final before anybody reads them
    self.reduce_scatter_piece(full_fp32, out_shard, rank * out_shard.numel())

  def adamw_allgather(self, tx, state, grad_shard: torch.Tensor, flat_param: torch.Tensor, pieces,
                      grad_scale: torch.Tensor) -> None:
    """Fused AdamW on this rank's shard + store of the new bf16 values into every rank's `flat_param`, one launch
    per piece `(flat start, length, offset in the shard tensors)`; closes with a barrier so no rank starts its
    next forward early."""
    from .. import optim
    count = int(state["count"]) + 1
    lr = optim._lr_at(tx._lr, count - 1)
    if isinstance(pieces, slice):
      pieces = [(pieces.start, grad_shard.numel(), 0)]
    ptrs = _ptr_array(self.ptrs_for(flat_param))
    ma, mu, nu = state["master"]["flat"], state["mu"]["flat"], state["nu"]["flat"]
    for lo, n, so in pieces:
      rc = self.lib.tx_adamw_allgather(
          ma.data_ptr() + 4 * so, mu.data_ptr() + 4 * so, nu.data_ptr() + 4 * so, grad_shard.data_ptr() + 4 * so, ptrs,
          lo, n, lr, tx.b1, tx.b2, tx.eps, tx.weight_decay, 1.0 - tx.b1 ** count, 1.0 - tx.b2 ** count,
          grad_scale.data_ptr(), self.world, self.rank, _lib.stream_ptr())
      _lib.check_rc(rc, "tx_adamw_allgather")
    self.barrier()      # all pushes have landed everywhere; also orders the next zeroing of gradients
    state["count"] = torch.tensor(count, dtype=torch.int32)
    if "hyperparams" in state:
      state["hyperparams"]["learning_rate"] = torch.tensor(optim._lr_at(tx._lr, count), dtype=torch.float32)

  def peer_copy_2d(self, src_ptr: int, dst: torch.Tensor, rows: int, cols: int, src_ld: int) -> None:
    rc = self.lib.tx_peer_copy_2d(src_ptr, dst.data_ptr(), rows, cols, src_ld, dst.stride(0), _lib.stream_ptr())
    _lib.check_rc(rc, "tx_peer_copy_2d")
