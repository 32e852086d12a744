"""What a launched process can ask of its runtime, independent of the platform.

A process body has the signature ``main(ctx: ProcessContext, argv: list[str])``.
``ctx.dist`` brings up ``torch.distributed`` (NCCL on GPUs, gloo on CPU) from
the launcher's environment; ``ctx.ipc.discovery`` lets processes find each other
by (id, port) before any collective exists.

Counterpart of tunix/experimental/distributed/runtime/context.py, whose
``jax`` member is replaced by ``dist``.
"""

from __future__ import annotations

from typing import Any, Callable


class DistContext:
  """Initialises and tears down the process group of this process."""

  def initialize(self, backend: str | None = None, **kwargs) -> None:
    pass

  def shutdown(self) -> None:
    pass

  @property
  def rank(self) -> int:
    return 0

  @property
  def world_size(self) -> int:
    return 1


class DiscoveryContext:
  """Peer registration: a server side (`on_register`) and a client side."""

  def on_register(self, callback: Callable[[str, int, bytes], None]) -> None:
    """`callback(hostname, port, metadata)` runs for every peer that registers."""

  def register(self, metadata: bytes) -> None:
    """Announces this process to every address it was told to register with."""


class IpcContext:

  @property
  def discovery(self) -> DiscoveryContext:
    return DiscoveryContext()


class ProcessContext:

  def __enter__(self) -> "ProcessContext":
    return self

  def __exit__(self, exc_type: Any, exc: Any, tb: Any) -> None:
    pass

  @property
  def dist(self) -> DistContext:
    return DistContext()

  @property
  def ipc(self) -> IpcContext:
    return IpcContext()
