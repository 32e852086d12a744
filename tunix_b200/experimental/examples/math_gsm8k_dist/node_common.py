"""What the three worker nodes share: serving a worker object, announcing it, and waiting for the end.

A node's announcement through discovery is one line of JSON: its role, its worker id, the port of its
remote-execution server and, for the two ends of weight transfers, the port of its host-staged endpoint and the
work unit that endpoint holds. Standalone (`python -m ...run_trainer_node`) a node runs under the local executor;
under the runtime launcher (`--process_main=...run_trainer_node.main`) it gets the launcher's context.
"""
from __future__ import annotations

import argparse
import json
import logging
import sys
import threading
from typing import Any, Dict, Optional, Sequence

from ...distributed.runtime import main as rt_main
from ...orchestrator import host_staged_handler, weight_sync
from ...worker import remote_execution

stop = threading.Event()              # set to end every node body of this OS process (tests, Ctrl-C)


def common_flags(parser: argparse.ArgumentParser, default_port: int) -> None:
  parser.add_argument("--model", default="tiny")
  parser.add_argument("--weights", default=None, help="local safetensors directory (random weights when absent)")
  parser.add_argument("--tokenizer", default=None, help="local Hugging Face tokenizer directory")
  parser.add_argument("--seed", type=int, default=0)
  parser.add_argument("--port", type=int, default=default_port, help="remote-execution port (0: any free port)")
  parser.add_argument("--host", default="127.0.0.1", help="address to serve on; 0.0.0.0 across machines")
  parser.add_argument("--worker_id", default=None)


def announcement(role: str, worker_id: str, rpc_port: int, staged: Optional[host_staged_handler.HostStagedEndpoint] = None,
                 unit: Optional[weight_sync.WorkUnitId] = None) -> bytes:
  info: Dict[str, Any] = {"role": role, "worker_id": worker_id, "rpc_port": int(rpc_port)}
  if staged is not None and unit is not None:
    info.update(staged_port=int(staged.address[1]),
                unit=[unit.job_name, unit.job_replica_id, int(unit.data_replica_idx)])
  return json.dumps(info).encode("utf-8")


def parse_announcement(metadata: bytes) -> Dict[str, Any]:
  info = json.loads(metadata.decode("utf-8"))
  if "unit" in info:
    job, replica, index = info["unit"]
    info["unit"] = weight_sync.WorkUnitId(job_name=job, job_replica_id=replica, data_replica_idx=int(index))
  return info


def serve_and_wait(ctx: Any, worker: Any, args: argparse.Namespace, role: str,
                   staged: Optional[host_staged_handler.HostStagedEndpoint] = None,
                   unit: Optional[weight_sync.WorkUnitId] = None) -> None:
  server = remote_execution.GrpcRemoteExecutionServer(worker)
  server.start_serving(args.port, args.host)
  logging.info("%s %s serving on %s:%d", role, worker.info().worker_id, args.host, server.port)
  try:
    if getattr(ctx.ipc.discovery, "_peers", None):
      ctx.ipc.discovery.register(announcement(role, worker.info().worker_id, server.port, staged, unit))
    stop.wait()
  finally:
    server.shutdown()
    if staged is not None:
      staged.close()


def run_standalone(process_main: str, argv: Sequence[str]) -> None:
  logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(message)s")
  try:
    rt_main.main([sys.argv[0], f"--process_main={process_main}", *argv])
  except KeyboardInterrupt:
    stop.set()
