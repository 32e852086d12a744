"""String-keyed class registries for agents and environments, with discovery.

`Registry.register` works as ``@reg.register("name")``, ``@reg.register()`` and
bare ``@reg.register``. `auto_discover_modules` imports every Python file under
the given packages or directories whose source (checked on the AST, without
running it) decorates a class with one of the registries, so user plug-ins
register themselves by being on the path.

Contract of tunix/experimental/rl/agentic/registry.py.
"""

from __future__ import annotations

import ast
import contextlib
import importlib
import importlib.util
import logging
import os
import sys
from typing import Any, Callable, Type, TypeVar

T = TypeVar("T")
log = logging.getLogger(__name__)


class Registry:

  def __init__(self, name: str = "Registry"):
    self.name = name
    self._registry: dict[str, Type[Any]] = {}

  def register(self, name_or_cls=None, *, override: bool = False):
    def put(key: str, cls):
      if key in self._registry and self._registry[key] is not cls and not override:
        raise ValueError(
            f"{self.name}: '{key}' is already registered to"
            f" {self._registry[key].__qualname__}")
      self._registry[key] = cls
      return cls

    if isinstance(name_or_cls, type):
      return put(name_or_cls.__name__, name_or_cls)
    if name_or_cls is not None and not isinstance(name_or_cls, str):
      raise TypeError(f"{self.name}: key must be a string, got {name_or_cls!r}")

    def decorator(cls: Type[T]) -> Type[T]:
      return put(name_or_cls or cls.__name__, cls)
    return decorator

  def get(self, name: str) -> Type[Any]:
    try:
      return self._registry[name]
    except KeyError:
      raise KeyError(
          f"{self.name}: '{name}' is not registered; known: {self.keys()}"
      ) from None

  def contains(self, name: str) -> bool:
    return name in self._registry

  def __contains__(self, name: str) -> bool:
    return name in self._registry

  def keys(self) -> list[str]:
    return sorted(self._registry)


AGENT_REGISTRY = Registry("AgentRegistry")
ENV_REGISTRY = Registry("EnvRegistry")
register_agent = AGENT_REGISTRY.register
register_env = ENV_REGISTRY.register

_REGISTRY_NAMES = {"register_agent", "register_env", "AGENT_REGISTRY",
                   "ENV_REGISTRY"}


def has_registry_decorator(file_path: str) -> bool:
  """True when a class in the file is decorated through a registry.

  Follows import aliases (``from ... import register_agent as ra``) and local
  assignments (``my = Registry("x")``, ``reg = AGENT_REGISTRY.register``).
  Unparseable files count as False.
  """
  try:
    with open(file_path, "r", encoding="utf-8") as f:
      tree = ast.parse(f.read(), filename=file_path)
  except (OSError, SyntaxError, ValueError):
    return False
  names = set(_REGISTRY_NAMES)
  for node in ast.walk(tree):
    if isinstance(node, ast.ImportFrom):
      mod = node.module or ""
      local = bool(node.level) or "agentic" in mod or mod.endswith("registry")
      for a in node.names:
        if a.name in names or (local and a.name in ("register", "registry")):
          names.add(a.asname or a.name)
    elif isinstance(node, ast.Import):
      for a in node.names:
        if "registry" in a.name and "agentic" in a.name:
          names.add(a.asname or a.name.split(".")[0])
    elif isinstance(node, ast.Assign):
      fn = node.value.func if isinstance(node.value, ast.Call) else node.value
      ident = getattr(fn, "id", None) or getattr(fn, "attr", None)
      base = getattr(getattr(fn, "value", None), "id", None)
      if ident in names or ident == "Registry" or base in names:
        names.update(t.id for t in node.targets if isinstance(t, ast.Name))
  for node in ast.walk(tree):
    if not isinstance(node, ast.ClassDef):
      continue
    for dec in node.decorator_list:
      fn = dec.func if isinstance(dec, ast.Call) else dec
      if getattr(fn, "id", None) in names or getattr(fn, "attr", None) in names:
        return True
      base = getattr(getattr(fn, "value", None), "id", None)
      if base in names and getattr(fn, "attr", None) == "register":
        return True
  return False


def _file_path_to_module_name(file_path: str) -> str | None:
  """Dotted name of a file that sits inside a package on sys.path, else None."""
  path = os.path.abspath(file_path)
  best = None
  for root in sys.path:
    root = os.path.abspath(root or os.getcwd())
    if path.startswith(root + os.sep):
      rel = os.path.relpath(path, root)
      if best is None or len(rel) < len(best):
        best = rel
  if best is None:
    return None
  parts = best[:-3].split(os.sep)
  if parts[-1] == "__init__":
    parts = parts[:-1]
  if not parts or not all(p.isidentifier() for p in parts):
    return None
  return ".".join(parts)


@contextlib.contextmanager
def _add_sys_path(path: str):
  added = path not in sys.path
  if added:
    sys.path.insert(0, path)
  try:
    yield
  finally:
    if added:
      with contextlib.suppress(ValueError):
        sys.path.remove(path)


def _iter_py_files(root: str):
  if os.path.isfile(root):
    yield root
    return
  for d, dirs, files in os.walk(root):
    dirs[:] = sorted(x for x in dirs if not x.startswith((".", "__pycache__")))
    for f in sorted(files):
      if f.endswith(".py"):
        yield os.path.join(d, f)


def auto_discover_modules(*package_or_directory_paths: str) -> list[str]:
  """Imports files that register agents or environments; returns their names.

  Each argument is a dotted package name or a filesystem path. A file that
  fails to import is logged and skipped.
  """
  imported = []
  for target in package_or_directory_paths:
    root = target
    if not os.path.exists(target):
      spec = importlib.util.find_spec(target)
      if spec is None:
        log.warning("auto_discover_modules: cannot find %s", target)
        continue
      root = (spec.submodule_search_locations[0]
              if spec.submodule_search_locations else spec.origin)
    root = os.path.abspath(root)
    for path in _iter_py_files(root):
      if not has_registry_decorator(path):
        continue
      name = _file_path_to_module_name(path)
      try:
        if name is not None:
          importlib.import_module(name)
        else:
          name = "_tunix_discovered_" + "".join(
              c if c.isalnum() else "_" for c in path)
          if name not in sys.modules:
            with _add_sys_path(os.path.dirname(path)):
              spec = importlib.util.spec_from_file_location(name, path)
              mod = importlib.util.module_from_spec(spec)
              sys.modules[name] = mod
              try:
                spec.loader.exec_module(mod)
              except BaseException:
                sys.modules.pop(name, None)
                raise
        imported.append(name)
      except Exception:  # pylint: disable=broad-exception-caught
        log.exception("auto_discover_modules: importing %s failed", path)
  return imported
