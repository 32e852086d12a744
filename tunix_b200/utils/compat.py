"""Small compatibility helpers (tunix/utils/compat.py): a module-list alias, a mesh context
manager, and a decorator that keeps a renamed constructor keyword working for one more release."""
from __future__ import annotations

import contextlib
import functools
import logging
from typing import Any, Callable

import torch

log = logging.getLogger(__name__)

ModuleList = torch.nn.ModuleList


@contextlib.contextmanager
def set_mesh(mesh):
  """`with set_mesh(m):` makes `m` the current mesh of `tunix_b200.dist.mesh` inside the block."""
  from ..dist import mesh as mesh_lib
  previous = mesh_lib.current_mesh()
  mesh_lib.set_current_mesh(mesh)
  try:
    yield mesh
  finally:
    mesh_lib.set_current_mesh(previous)


def alias_init_param(old_name: str, new_name: str) -> Callable[[Callable[..., Any]], Callable[..., Any]]:
  """`@alias_init_param("rl_cluster", "rl_engine")` lets callers keep passing the old keyword: it is
  forwarded under the new name with a deprecation warning; passing both is an error."""
  def wrap(init: Callable[..., Any]) -> Callable[..., Any]:
    @functools.wraps(init)
    def __init__(self, *args, **kwargs):
      if old_name in kwargs:
        if new_name in kwargs:
          raise ValueError(f"pass '{new_name}' only, not both '{new_name}' and its old spelling '{old_name}'")
        log.warning("keyword '%s' is deprecated, use '%s'", old_name, new_name)
        kwargs[new_name] = kwargs.pop(old_name)
      return init(self, *args, **kwargs)
    return __init__
  return wrap
