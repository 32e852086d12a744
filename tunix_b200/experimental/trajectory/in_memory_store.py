"""Process-local trajectory store for tests and single-process runs.

Same contract as tunix/experimental/trajectory/in_memory_store.py.
"""

from __future__ import annotations

import threading

from . import store
from . import trajectory as trajectory_lib


class InMemoryTrajectoryStore(store.TrajectoryReader, store.TrajectoryWriter):

  def __init__(self, trajectory_cls=trajectory_lib.Trajectory) -> None:
    self._lock = threading.Lock()
    self._metadata: dict[str, trajectory_lib.TrajectoryMetadata] = {}
    self._steps: dict[str, dict[int, trajectory_lib.Step]] = {}
    self._trajectory_cls = trajectory_cls

  def get_trajectories_metadata(self):
    with self._lock:
      return [m.model_copy(deep=True) for m in self._metadata.values()]

  def get_trajectories(self, trajectory_ids):
    out = []
    with self._lock:
      for tid in trajectory_ids:
        if tid not in self._steps and tid not in self._metadata:
          raise store.TrajectoryNotFoundError(tid)
        if tid not in self._metadata:
          raise store.TrajectoryMetadataNotFoundError(tid)
        meta = self._metadata[tid].model_dump()
        steps = [s.model_copy(deep=True)
                 for _, s in sorted(self._steps.get(tid, {}).items())]
        out.append(self._trajectory_cls(**meta, steps=steps))
    return out

  def add_step(self, step, metadata) -> None:
    tid = store.validate_trajectory_id(metadata.trajectory_id)
    with self._lock:
      self._metadata[tid] = metadata.model_copy(deep=True)
      self._steps.setdefault(tid, {})[step.step_id] = step.model_copy(deep=True)

  def update_metadata(self, metadata) -> None:
    tid = store.validate_trajectory_id(metadata.trajectory_id)
    with self._lock:
      self._metadata[tid] = metadata.model_copy(deep=True)
      self._steps.setdefault(tid, {})

  def flush(self) -> None:
    pass
