"""Objects that freeze when their construction is complete (the role of tunix/utils/immutable.py:20-48).

`FrozenAfterInit` is a mixin, not a metaclass: `__init_subclass__` wraps every constructor defined along the class
hierarchy so that each counts its nesting on the instance; when the outermost constructor returns, attribute
assignment and deletion are locked. Subclass constructors therefore initialise their fields normally, in any order
relative to `super().__init__()`, and an instance shared between threads or episodes cannot be changed afterwards.
`thaw()` is the explicit, visible escape for code that owns an instance (tests, rebuilding a tool in place)."""
from __future__ import annotations

import contextlib
import functools
from typing import Any, Callable


class FrozenAfterInit:
  _ctor_depth = 0
  _frozen = False

  def __init_subclass__(cls, **kwargs):
    super().__init_subclass__(**kwargs)
    if "__init__" in cls.__dict__:
      cls.__init__ = _counting(cls.__dict__["__init__"])

  def __init__(self, *args, **kwargs):
    super().__init__(*args, **kwargs)
    if self._ctor_depth == 0:                 # constructed directly, no wrapped constructor around this call
      object.__setattr__(self, "_frozen", True)

  def __setattr__(self, name: str, value: Any) -> None:
    if self._frozen:
      raise AttributeError(f"Cannot modify immutable {type(self).__name__} instance after initialization "
                           f"(attempted to set '{name}')")
    object.__setattr__(self, name, value)

  def __delattr__(self, name: str) -> None:
    if self._frozen:
      raise AttributeError(f"Cannot modify immutable {type(self).__name__} instance after initialization "
                           f"(attempted to delete '{name}')")
    object.__delattr__(self, name)

  @contextlib.contextmanager
  def thaw(self):
    """Assignment is allowed inside the block."""
    object.__setattr__(self, "_frozen", False)
    try:
      yield self
    finally:
      object.__setattr__(self, "_frozen", True)


def _counting(init: Callable[..., None]) -> Callable[..., None]:
  @functools.wraps(init)
  def wrapped(self, *args, **kwargs):
    object.__setattr__(self, "_ctor_depth", self._ctor_depth + 1)
    try:
      init(self, *args, **kwargs)
    finally:
      object.__setattr__(self, "_ctor_depth", self._ctor_depth - 1)
      if self._ctor_depth == 0:
        object.__setattr__(self, "_frozen", True)
  return wrapped
