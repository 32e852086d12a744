"""Rollout process of the toy RL system (tunix/experimental/distributed/examples/rl/rollout.py): serves
`RolloutService.generate` and announces itself to the orchestrator. See `orchestrator` for the command line."""
import argparse
import logging
import threading

from . import services

stop = threading.Event()          # set by a host program (or a test) to end every serving body of this process


def main(ctx, argv) -> None:
  parser = argparse.ArgumentParser()
  parser.add_argument("--message", type=str, default="this is rollout!")
  parser.add_argument("--server_id", type=str, default="rollout")
  parser.add_argument("--server_port", type=int, default=11111)
  parser.add_argument("--seed", type=int, default=0)
  args = parser.parse_args(argv)
  logging.info(args.message)
  server = services.serve(services.RolloutService(args.server_id, args.seed), args.server_port)
  try:
    ctx.ipc.discovery.register(services.announce("rollout", server.port, args.server_id))
    logging.info("rollout %s serving on port %d", args.server_id, server.port)
    stop.wait()
  finally:
    server.shutdown()
