"""Runs process bodies on this host; peers are reached over 127.0.0.1
(tunix/experimental/distributed/runtime/executors/local_executor.py)."""
from __future__ import annotations

from ..contexts import local_context

LocalProcessContext = local_context.LocalProcessContext
TorchDistContext = local_context.TorchDistContext


class LocalExecutor:
  """`run(main_fn, argv, context_args)` inside a process context that lives exactly as long as the body."""

  context_cls = local_context.LocalProcessContext

  def run(self, main_fn, argv, context_args):
    with self.context_cls(context_args) as ctx:
      return main_fn(ctx, argv)
