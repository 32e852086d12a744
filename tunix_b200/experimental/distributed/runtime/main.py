"""Launcher: runs one or several logical processes under one executor.

  python -m tunix_b200.experimental.distributed.runtime.main \
      --process_main=pkg.module.main --flag=value

  python -m tunix_b200.experimental.distributed.runtime.main \
      --process --process_main=a.main --discovery_id=door --discovery_port=12345 \
      --process --process_main=b.main --discovery_addrs=door:12345

A "process" here is a logical one: several given in one invocation run as
threads of this OS process and share the executor. Flags the launcher does not
know are passed to the body untouched. A non-zero `SystemExit` from any body
ends the whole OS process with that code, so an orchestration layer restarts
the group rather than waiting on the survivors.

Counterpart of tunix/experimental/distributed/runtime/main.py.
"""

from __future__ import annotations

import argparse
import concurrent.futures
import dataclasses
import importlib
import logging
import os
import sys
from typing import Any, Callable

DEFAULT_EXECUTOR = (
    "tunix_b200.experimental.distributed.runtime.executor.LocalExecutor")


@dataclasses.dataclass(frozen=True)
class PreparedProcess:
  main_fn: Callable[..., Any]
  argv: list[str]
  context_args: argparse.Namespace


def import_symbol(fqn: str) -> Any:
  """Resolves ``pkg.mod.attr`` (or ``pkg.mod:attr``) to the object."""
  if not fqn:
    raise ValueError("empty symbol name")
  mod_name, sep, attr = fqn.replace(":", ".").rpartition(".")
  if not sep:
    raise ValueError(f"'{fqn}' is not a fully qualified name")
  return getattr(importlib.import_module(mod_name), attr)


def split_process_argv(argv: list[str]) -> list[list[str]]:
  if "--process" not in argv:
    return [argv]
  out, cur = [], []
  for tok in argv:
    if tok == "--process":
      if cur:
        out.append(cur)
      cur = []
    else:
      cur.append(tok)
  if cur:
    out.append(cur)
  return out


def prepare_process(argv: list[str]) -> PreparedProcess:
  p = argparse.ArgumentParser(allow_abbrev=False, add_help=False)
  p.add_argument("--process_main", type=str, default="")
  p.add_argument("--discovery_id", type=str, default="")
  p.add_argument("--discovery_port", type=int, default=0)
  p.add_argument("--discovery_addrs", type=str, default="")
  ctx_args, rest = p.parse_known_args(argv)
  try:
    fn = import_symbol(ctx_args.process_main)
  except (AttributeError, ImportError, ValueError) as e:
    raise ValueError(
        f"Invalid --process_main={ctx_args.process_main}: {e}") from e
  return PreparedProcess(fn, rest, ctx_args)


def main(argv: list[str]) -> None:
  p = argparse.ArgumentParser(allow_abbrev=False, add_help=False)
  p.add_argument("--process_executor", type=str, default=DEFAULT_EXECUTOR)
  main_args, rest = p.parse_known_args(argv)
  rest = rest[1:]
  executor = import_symbol(main_args.process_executor)()
  logging.basicConfig(
      level=logging.INFO, force=True,
      format="%(asctime)s [%(filename)s:%(lineno)d] %(levelname)s %(message)s")
  prepared = [prepare_process(a) for a in split_process_argv(rest)]
  if len(prepared) == 1:
    one = prepared[0]
    executor.run(one.main_fn, one.argv, one.context_args)
    return
  with concurrent.futures.ThreadPoolExecutor(len(prepared)) as pool:
    futs = [pool.submit(executor.run, q.main_fn, q.argv, q.context_args)
            for q in prepared]
    try:
      for f in concurrent.futures.as_completed(futs):
        f.result()
    except SystemExit as e:
      code = e.code if isinstance(e.code, int) else (0 if e.code is None else 1)
      if code != 0:
        logging.error("a process exited with code %d; ending the group", code)
        logging.shutdown()
        os._exit(code)
    except BaseException:
      logging.exception("a process raised; ending the group")
      logging.shutdown()
      os._exit(1)


if __name__ == "__main__":
  main(sys.argv)
