"""Client side of the worker-transport example
(tunix/experimental/distributed/examples/worker_transport/transport.py): a `Worker` whose every method is a remote
call on a handle, so that an orchestrator written against the `Worker` interface drives a worker in another process
without knowing it."""
from __future__ import annotations

from typing import Any

from ....common import datatypes
from ....worker import abstract_worker, remote_execution


class RemoteWorker(abstract_worker.Worker):

  def __init__(self, address_or_handle: Any):
    self._handle = (address_or_handle if isinstance(address_or_handle, remote_execution.ActorHandle)
                    else remote_execution.ActorHandle.from_address(address_or_handle))

  @property
  def state(self) -> datatypes.WorkerState:              # the truth lives on the other side
    return self.heartbeat().state

  def initialize(self) -> datatypes.Response:
    return self._handle.submit("initialize")

  def compile(self, dummy_data: Any = None) -> datatypes.Response:
    return self._handle.submit("compile", dummy_data)

  def start(self) -> datatypes.Response:
    return self._handle.submit("start")

  def stop(self) -> datatypes.Response:
    return self._handle.submit("stop")

  def info(self) -> datatypes.WorkerInfo:
    return self._handle.submit("info")

  def heartbeat(self) -> datatypes.HealthReport:
    return self._handle.submit("heartbeat")

  def call(self, method: str, *args, **kwargs) -> Any:
    """Anything beyond the lifecycle (generate, train_step, ...)."""
    return self._handle.submit(method, *args, **kwargs)
