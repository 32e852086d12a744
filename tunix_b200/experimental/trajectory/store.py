"""Trajectory store protocols (tunix/experimental/trajectory/store.py)."""

from __future__ import annotations

import typing
from typing import Protocol

from . import trajectory as trajectory_lib


class TrajectoryNotFoundError(KeyError):

  def __init__(self, trajectory_id: str) -> None:
    super().__init__(f"Trajectory '{trajectory_id}' not found")
    self.trajectory_id = trajectory_id


class TrajectoryMetadataNotFoundError(KeyError):

  def __init__(self, trajectory_id: str) -> None:
    super().__init__(f"Metadata for trajectory '{trajectory_id}' not found")
    self.trajectory_id = trajectory_id


def validate_trajectory_id(trajectory_id: str | None) -> str:
  """A usable id: a non-empty string that is a single safe path component."""
  if not isinstance(trajectory_id, str) or not trajectory_id:
    raise ValueError("trajectory_id must be a non-empty string")
  if trajectory_id in (".", "..") or any(
      c in trajectory_id for c in ("/", "\\", "\0")):
    raise ValueError(
        f"trajectory_id {trajectory_id!r} must be a single path component")
  return trajectory_id


@typing.runtime_checkable
class TrajectoryReader(Protocol):

  def get_trajectories_metadata(
      self) -> list[trajectory_lib.TrajectoryMetadata]:
    ...

  def get_trajectories(
      self, trajectory_ids: list[str]) -> list[trajectory_lib.Trajectory]:
    ...


@typing.runtime_checkable
class TrajectoryWriter(Protocol):
  """Writers snapshot what they are given; callers may keep mutating it."""

  def add_step(self, step: trajectory_lib.Step,
               metadata: trajectory_lib.TrajectoryMetadata) -> None:
    ...

  def update_metadata(self,
                      metadata: trajectory_lib.TrajectoryMetadata) -> None:
    ...

  def flush(self) -> None:
    ...
