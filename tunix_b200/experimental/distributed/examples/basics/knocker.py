"""Discovery, client side: registers with the door and says something
(tunix/experimental/distributed/examples/basics/knocker.py). See `door` for the command line."""
import argparse
import logging


def main(ctx, argv) -> None:
  parser = argparse.ArgumentParser()
  parser.add_argument("--message", type=str, default="this is knocker!")
  parser.add_argument("--say", type=str, default="")
  args = parser.parse_args(argv)
  logging.info(args.message)
  ctx.ipc.discovery.register(args.say.encode("utf-8"))
