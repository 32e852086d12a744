"""Directory-backed trajectory store.

Layout: ``<root>/<trajectory_id>/metadata.json`` plus one
``step_<id, 6 digits>.json`` per step; embedded sub-agents are not split out.
Writes go through `AsyncFileWriter`; reads list the directory, so several
processes may write different trajectories under one root while another reads.

Contract of tunix/experimental/trajectory/file_store.py.
"""

from __future__ import annotations

import json
import os
import re

from . import async_writer
from . import store
from . import trajectory as trajectory_lib

_STEP_RE = re.compile(r"^step_(\d+)\.json$")


class FileTrajectoryStore(store.TrajectoryReader, store.TrajectoryWriter):

  def __init__(self, root_dir: str,
               trajectory_cls=trajectory_lib.Trajectory,
               writer: async_writer.AsyncFileWriter | None = None) -> None:
    self._root = os.fspath(root_dir)
    self._trajectory_cls = trajectory_cls
    self._writer = writer or async_writer.AsyncFileWriter()

  @property
  def root_dir(self) -> str:
    return self._root

  def get_trajectory_dir(self, trajectory_id: str) -> str:
    return os.path.join(self._root, store.validate_trajectory_id(trajectory_id))

  def get_trajectory_metadata_path(self, trajectory_id: str) -> str:
    return os.path.join(self.get_trajectory_dir(trajectory_id), "metadata.json")

  def get_step_path(self, trajectory_id: str, step_id: int) -> str:
    return os.path.join(self.get_trajectory_dir(trajectory_id),
                        f"step_{int(step_id):06d}.json")

  # -- reader -----------------------------------------------------------------

  def _metadata_cls(self):
    for base in self._trajectory_cls.__mro__[1:]:
      if issubclass(base, trajectory_lib.TrajectoryMetadata):
        return base
    return trajectory_lib.TrajectoryMetadata

  def _read_json(self, path):
    with open(path, "r", encoding="utf-8") as f:
      return json.load(f)

  def get_trajectories_metadata(self):
    if not os.path.isdir(self._root):
      return []
    out = []
    cls = self._metadata_cls()
    for name in sorted(os.listdir(self._root)):
      path = os.path.join(self._root, name, "metadata.json")
      if os.path.isfile(path):
        out.append(cls.model_validate(self._read_json(path)))
    return out

  def get_trajectories(self, trajectory_ids):
    out = []
    for tid in trajectory_ids:
      d = self.get_trajectory_dir(tid)
      if not os.path.isdir(d):
        raise store.TrajectoryNotFoundError(tid)
      mpath = os.path.join(d, "metadata.json")
      if not os.path.isfile(mpath):
        raise store.TrajectoryMetadataNotFoundError(tid)
      meta = self._read_json(mpath)
      steps = []
      for name in sorted(os.listdir(d)):
        if _STEP_RE.match(name):
          steps.append(self._read_json(os.path.join(d, name)))
      out.append(self._trajectory_cls.model_validate({**meta, "steps": steps}))
    return out

  # -- writer -----------------------------------------------------------------

  def add_step(self, step, metadata) -> None:
    tid = store.validate_trajectory_id(metadata.trajectory_id)
    self._writer.write_step(
        trajectory_id=tid, trajectory_dir=self.get_trajectory_dir(tid),
        metadata_path=self.get_trajectory_metadata_path(tid), metadata=metadata,
        step_path=self.get_step_path(tid, step.step_id), step=step)

  def update_metadata(self, metadata) -> None:
    tid = store.validate_trajectory_id(metadata.trajectory_id)
    self._writer.write_step(
        trajectory_id=tid, trajectory_dir=self.get_trajectory_dir(tid),
        metadata_path=self.get_trajectory_metadata_path(tid), metadata=metadata)

  def flush(self) -> None:
    self._writer.flush()

  def close(self) -> None:
    self._writer.close()
