"""Discovery, client side: registers with the door and says something
(tunix/experimental/distributed/examples/basics/knocker.py). See `door` for the command line."""
import logging

from . import _flags


def main(ctx, argv) -> int:
  words = _flags.value(argv, "--say").encode("utf-8")
  logging.info(_flags.value(argv, "--message", "this is knocker!"))
  ctx.ipc.discovery.register(words)
  return len(words)
