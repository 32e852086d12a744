"""A body with its own flag: everything after the launcher's flags reaches it untouched
(tunix/experimental/distributed/examples/basics/flag.py).

  python -m tunix_b200.experimental.distributed.runtime.main \\
      --process_main=tunix_b200.experimental.distributed.examples.basics.flag.main --message="hi there"
"""
from . import _flags


def main(ctx, argv) -> str:
  text = _flags.value(argv, "--message")
  print(text)
  return text
