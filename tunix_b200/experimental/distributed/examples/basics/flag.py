"""A body with its own flag: everything after the launcher's flags reaches it untouched
(tunix/experimental/distributed/examples/basics/flag.py).

  python -m tunix_b200.experimental.distributed.runtime.main \\
      --process_main=tunix_b200.experimental.distributed.examples.basics.flag.main --message="hi there"
"""
import argparse


def main(ctx, argv) -> None:
  parser = argparse.ArgumentParser()
  parser.add_argument("--message", type=str, default="")
  print(parser.parse_args(argv).message)
