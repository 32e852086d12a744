"""Runs process bodies on this host; peers are reached over 127.0.0.1."""

from __future__ import annotations

import os

from .. import context
from .. import discovery


class TorchDistContext(context.DistContext):
  """Process group from the launcher's RANK / WORLD_SIZE / MASTER_* variables."""

  def __init__(self, default_addr: str = "127.0.0.1"):
    self._default_addr = default_addr
    self._owned = False

  def initialize(self, backend: str | None = None, **kwargs) -> None:
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


class _Ipc(context.IpcContext):

  def __init__(self, disc):
    self._disc = disc

  @property
  def discovery(self):
    return self._disc


class LocalProcessContext(context.ProcessContext):

  _HOST = "127.0.0.1"

  def __init__(self, context_args):
    self._disc = discovery.TcpDiscovery(
        getattr(context_args, "discovery_id", "") or "local",
        getattr(context_args, "discovery_port", 0),
        getattr(context_args, "discovery_addrs", ""),
        bind_host=self._bind_host(), resolve=self._resolve)
    self._dist = TorchDistContext(self._HOST)
    self._ipc = _Ipc(self._disc)

  def _bind_host(self) -> str:
    return self._HOST

  def _resolve(self, host: str) -> str:
    return self._HOST   # discovery ids are names, not hosts, on one machine

  def __enter__(self):
    self._disc.start()
    return self

  def __exit__(self, exc_type, exc, tb) -> None:
    self._disc.stop()
    self._dist.shutdown()

  @property
  def dist(self):
    return self._dist

  @property
  def ipc(self):
    return self._ipc


class LocalExecutor:
  """`run(main_fn, argv, context_args)` inside a `LocalProcessContext`."""

  context_cls = LocalProcessContext

  def run(self, main_fn, argv, context_args):
    with self.context_cls(context_args) as ctx:
      return main_fn(ctx, argv)
