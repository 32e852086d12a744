"""Trainer process of the toy RL system (tunix/experimental/distributed/examples/rl/trainer.py): serves
`TrainerService.train` and announces itself to the orchestrator. See `orchestrator` for the command line."""
import argparse
import logging

from . import services
from .rollout import stop


def main(ctx, argv) -> None:
  parser = argparse.ArgumentParser()
  parser.add_argument("--message", type=str, default="this is trainer!")
  parser.add_argument("--server_port", type=int, default=22222)
  args = parser.parse_args(argv)
  logging.info(args.message)
  server = services.serve(services.TrainerService(), args.server_port)
  try:
    ctx.ipc.discovery.register(services.announce("trainer", server.port, "trainer"))
    logging.info("trainer serving on port %d", server.port)
    stop.wait()
  finally:
    server.shutdown()
