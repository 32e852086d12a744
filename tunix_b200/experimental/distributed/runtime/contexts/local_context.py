"""Process context for bodies that all run on this machine
(tunix/experimental/distributed/runtime/contexts/local_context.py:27-159).

Discovery ids are names, not hosts: every id resolves to the loopback address and only the port tells two
processes apart. The process group comes from the launcher's RANK / WORLD_SIZE / MASTER_* variables, with
loopback defaults for a single process.
"""
from __future__ import annotations

import os
from typing import Any, Optional

from .. import context, discovery

LOOPBACK = "127.0.0.1"


def resolve_discovery_address(discovery_address: str) -> str:
  """'door:12345' -> '127.0.0.1:12345': on one machine the id part only names the peer."""
  _, _, port = discovery_address.rpartition(":")
  if not port.isdigit():
    raise ValueError(f"discovery address '{discovery_address}' is not id:port")
  return f"{LOOPBACK}:{port}"


class TorchDistContext(context.DistContext):
  """Process group from the launcher's RANK / WORLD_SIZE / MASTER_* variables."""

  def __init__(self, default_addr: str = LOOPBACK):
    self._default_addr = default_addr
    self._owned = False

  def initialize(self, backend: Optional[str] = None, **kwargs) -> None:
    import torch
    import torch.distributed as dist
    if dist.is_initialized():
      return
    os.environ.setdefault("MASTER_ADDR", self._default_addr)
    os.environ.setdefault("MASTER_PORT", "29500")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    if backend is None:
      backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
      torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group(backend=backend, **kwargs)
    self._owned = True

  def shutdown(self) -> None:
    import torch.distributed as dist
    if self._owned and dist.is_initialized():
      dist.destroy_process_group()
    self._owned = False

  @property
  def rank(self) -> int:
    return int(os.environ.get("RANK", "0"))

  @property
  def world_size(self) -> int:
    return int(os.environ.get("WORLD_SIZE", "1"))


class LocalIpcContext(context.IpcContext):
  """Owns the discovery endpoint: entering starts its listener (when a port was given), leaving stops it."""

  def __init__(self, disc: discovery.TcpDiscovery):
    self._disc = disc

  def __enter__(self) -> "LocalIpcContext":
    self._disc.start()
    return self

  def __exit__(self, exc_type: Any, exc: Any, tb: Any) -> None:
    self._disc.stop()

  @property
  def discovery(self) -> discovery.TcpDiscovery:
    return self._disc


class LocalProcessContext(context.ProcessContext):

  ipc_cls = LocalIpcContext

  def __init__(self, context_args: Any):
    self._disc = discovery.TcpDiscovery(
        self._own_name(getattr(context_args, "discovery_id", "") or "local"),
        getattr(context_args, "discovery_port", 0), getattr(context_args, "discovery_addrs", ""),
        bind_host=self._bind_host(), resolve=self._resolve)
    self._dist = TorchDistContext(LOOPBACK)
    self._ipc = self.ipc_cls(self._disc)

  def _own_name(self, discovery_id: str) -> str:
    """The name this process announces to the peers it registers with."""
    return discovery_id

  def _bind_host(self) -> str:
    return LOOPBACK

  def _resolve(self, host: str) -> str:
    return LOOPBACK

  def __enter__(self) -> "LocalProcessContext":
    self._ipc.__enter__()
    return self

  def __exit__(self, exc_type: Any, exc: Any, tb: Any) -> None:
    self._ipc.__exit__(exc_type, exc, tb)
    self._dist.shutdown()

  @property
  def dist(self) -> TorchDistContext:
    return self._dist

  @property
  def ipc(self) -> LocalIpcContext:
    return self._ipc
