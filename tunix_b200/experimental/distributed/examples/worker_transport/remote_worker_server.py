"""Server side of the worker-transport example
(tunix/experimental/distributed/examples/worker_transport/remote_worker_server.py): a process body that serves one
worker and announces its port.

  python -m tunix_b200.experimental.distributed.runtime.main \\
      --process_main=tunix_b200.experimental.distributed.examples.worker_transport.remote_worker_server.main \\
      --worker_id=remote-0 --port=50061

and, from the orchestrating process:

  from tunix_b200.experimental.distributed.examples.worker_transport import transport
  worker = transport.RemoteWorker("grpc://127.0.0.1:50061")
  worker.initialize(); worker.compile(); worker.start(); print(worker.heartbeat())
"""
import argparse
import logging
import threading

from ....worker import remote_execution
from . import worker as worker_lib

stop = threading.Event()


def main(ctx, argv) -> None:
  parser = argparse.ArgumentParser()
  parser.add_argument("--worker_id", type=str, default="remote-0")
  parser.add_argument("--port", type=int, default=50061)
  parser.add_argument("--host", type=str, default="127.0.0.1")
  args = parser.parse_args(argv)
  server = remote_execution.GrpcRemoteExecutionServer(worker_lib.build(args.worker_id))
  server.start_serving(args.port, args.host)
  logging.info("worker %s served on %s:%d", args.worker_id, args.host, server.port)
  try:
    if getattr(ctx.ipc.discovery, "_peers", None):
      ctx.ipc.discovery.register(f"{args.worker_id}:{server.port}".encode())
    stop.wait()
  finally:
    server.shutdown()
