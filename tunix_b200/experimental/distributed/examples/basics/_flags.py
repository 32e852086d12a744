"""Flag reading for the one-flag example bodies: `value(argv, "--say", "")` accepts `--say=x` and `--say x`."""
from typing import Sequence


def value(argv: Sequence[str], name: str, default: str = "") -> str:
  found = default
  for position, token in enumerate(argv):
    if token == name and position + 1 < len(argv):
      found = argv[position + 1]
    elif token.startswith(name + "="):
      found = token[len(name) + 1:]
  return found
