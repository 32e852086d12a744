"""Launcher: runs one or several logical processes under one executor.

  python -m tunix_b200.experimental.distributed.runtime.main \
      --process_main=pkg.module.main --flag=value

  python -m tunix_b200.experimental.distributed.runtime.main \
      --process --process_main=a.main --discovery_id=door --discovery_port=12345 \
      --process --process_main=b.main --discovery_addrs=door:12345

A "process" here is a logical one: several given in one invocation run as threads of this OS process and share
the executor. The command line is read in two passes: `LaunchPlan.from_argv` takes the launcher's own flag
(`--process_executor`), cuts the rest at every `--process` marker and resolves each section's `--process_main`
plus discovery flags; whatever a section's parser does not know goes to the process body untouched. `run_group`
then starts the bodies and applies the group policy: the first body that leaves with a non-zero `SystemExit`, or
raises, ends the whole OS process with that code, so an orchestration layer restarts the group rather than waiting
on the survivors.

Counterpart of tunix/experimental/distributed/runtime/main.py.
"""

from __future__ import annotations

import argparse
import dataclasses
import importlib
import logging
import os
import sys
import threading
from typing import Any, Callable, List, Optional, Sequence

DEFAULT_EXECUTOR = "tunix_b200.experimental.distributed.runtime.executor.LocalExecutor"
PROCESS_MARKER = "--process"
_LOG_FORMAT = "%(asctime)s [%(filename)s:%(lineno)d] %(levelname)s %(message)s"


def import_symbol(fqn: str) -> Any:
  """Resolves ``pkg.mod.attr`` (or ``pkg.mod:attr``) to the object."""
  if not fqn:
    raise ValueError("empty symbol name")
  module, dot, attr = fqn.replace(":", ".").rpartition(".")
  if not dot:
    raise ValueError(f"'{fqn}' is not a fully qualified name")
  return getattr(importlib.import_module(module), attr)


def split_process_argv(argv: Sequence[str]) -> List[List[str]]:
  """Sections of the command line between `--process` markers (the whole line when there is no marker)."""
  if PROCESS_MARKER not in argv:
    return [list(argv)]
  sections: List[List[str]] = [[]]
  for tok in argv:
    if tok == PROCESS_MARKER:
      sections.append([])
    else:
      sections[-1].append(tok)
  return [s for s in sections if s]


def _context_parser() -> argparse.ArgumentParser:
  p = argparse.ArgumentParser(allow_abbrev=False, add_help=False)
  p.add_argument("--process_main", type=str, default="")
  p.add_argument("--discovery_id", type=str, default="")
  p.add_argument("--discovery_port", type=int, default=0)
  p.add_argument("--discovery_addrs", type=str, default="")
  return p


@dataclasses.dataclass(frozen=True)
class PreparedProcess:
  main_fn: Callable[..., Any]
  argv: List[str]
  context_args: argparse.Namespace


def prepare_process(argv: Sequence[str]) -> PreparedProcess:
  context_args, body_argv = _context_parser().parse_known_args(list(argv))
  try:
    body = import_symbol(context_args.process_main)
  except (AttributeError, ImportError, ValueError) as e:
    raise ValueError(f"Invalid --process_main={context_args.process_main}: {e}") from e
  return PreparedProcess(body, body_argv, context_args)


@dataclasses.dataclass
class LaunchPlan:
  executor: Any
  processes: List[PreparedProcess]

  @classmethod
  def from_argv(cls, argv: Sequence[str]) -> "LaunchPlan":
    p = argparse.ArgumentParser(allow_abbrev=False, add_help=False)
    p.add_argument("--process_executor", type=str, default=DEFAULT_EXECUTOR)
    own, rest = p.parse_known_args(list(argv))
    return cls(executor=import_symbol(own.process_executor)(),
               processes=[prepare_process(section) for section in split_process_argv(rest[1:])])   # rest[0]: program


def _exit_code(exit_: SystemExit) -> int:
  if isinstance(exit_.code, int):
    return exit_.code
  return 0 if exit_.code is None else 1


def run_group(plan: LaunchPlan) -> None:
  """One body: runs on the calling thread. Several: one thread each; the first failure ends the OS process."""
  if len(plan.processes) == 1:
    only = plan.processes[0]
    plan.executor.run(only.main_fn, only.argv, only.context_args)
    return
  failed = threading.Event()
  verdict: List[Optional[int]] = [None]

  def body(proc: PreparedProcess) -> None:
    try:
      plan.executor.run(proc.main_fn, proc.argv, proc.context_args)
    except SystemExit as e:
      if _exit_code(e) != 0 and verdict[0] is None:
        logging.error("a process exited with code %d; ending the group", _exit_code(e))
        verdict[0] = _exit_code(e)
        failed.set()
    except BaseException:     # noqa: BLE001
      logging.exception("a process raised; ending the group")
      if verdict[0] is None:
        verdict[0] = 1
      failed.set()

  threads = [threading.Thread(target=body, args=(proc,), name=f"process-{i}", daemon=True)
             for i, proc in enumerate(plan.processes)]
  for t in threads:
    t.start()
  while any(t.is_alive() for t in threads):
    if failed.wait(timeout=0.05):
      logging.shutdown()
      os._exit(verdict[0] or 1)
  if failed.is_set():
    logging.shutdown()
    os._exit(verdict[0] or 1)


def main(argv: Sequence[str]) -> None:
  plan = LaunchPlan.from_argv(argv)
  logging.basicConfig(level=logging.INFO, force=True, format=_LOG_FORMAT)
  run_group(plan)


if __name__ == "__main__":
  main(sys.argv)
