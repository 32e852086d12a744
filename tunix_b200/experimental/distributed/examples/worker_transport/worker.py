"""The object that is served in the worker-transport example
(tunix/experimental/distributed/examples/worker_transport/worker.py): a `MockWorker` is enough to show lifecycle
calls, replies and remote errors crossing a process boundary."""
from ....worker import mock_worker


def build(worker_id: str = "remote-0", roles=("rollout",), fail_in=()) -> mock_worker.MockWorker:
  return mock_worker.MockWorker(worker_id, roles, fail_in=fail_in)
