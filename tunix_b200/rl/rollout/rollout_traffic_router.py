"""Chooses the replica that serves a generate() call (tunix/rl/rollout/rollout_traffic_router.py:24-36)."""
from __future__ import annotations

import itertools
import threading
from typing import Any


class RolloutTrafficRouter:
  """Round-robin over `num_engines` replicas; thread-safe."""

  def __init__(self, num_engines: int):
    self.num_engines = num_engines
    self._it = itertools.cycle(range(num_engines))
    self._lock = threading.Lock()

  def route(self, request: Any) -> int:
    with self._lock:
      return next(self._it)
