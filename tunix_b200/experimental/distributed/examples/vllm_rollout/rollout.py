"""Rollout process of the generation-load example
(tunix/experimental/distributed/examples/vllm_rollout/rollout.py): serves a `RolloutWorker` and announces
`worker id | port | model` to the orchestrator.

`--engine vllm` serves the installed vLLM in process (its own CUDA kernels; needs a GPU); the default `native` is
this framework's paged engine, which also runs on a CPU with `--model tiny`. See `orchestrator` for the command line.
"""
from __future__ import annotations

import argparse
import logging
import threading

from ....examples.math_gsm8k_dist import node_common, run_rollout_node
from ....worker import remote_execution

stop = threading.Event()


def main(ctx, argv) -> None:
  parser = argparse.ArgumentParser()
  node_common.common_flags(parser, default_port=50081)
  parser.add_argument("--engine", choices=("native", "vllm"), default="native")
  parser.add_argument("--page_size", type=int, default=16)
  parser.add_argument("--max_batch", type=int, default=64)
  parser.add_argument("--max_seq_len", type=int, default=1024)
  args = parser.parse_args(argv)
  args.agentic = False
  worker, endpoint, _ = run_rollout_node.build_worker(args)
  worker.initialize()
  server = remote_execution.GrpcRemoteExecutionServer(worker)
  server.start_serving(args.port, args.host)
  try:
    ctx.ipc.discovery.register(f"{worker.info().worker_id}|{server.port}|{args.model}".encode("utf-8"))
    logging.info("rollout %s (%s engine, model %s) on port %d", worker.info().worker_id, args.engine, args.model, server.port)
    stop.wait()
  finally:
    server.shutdown()
    endpoint.close()
