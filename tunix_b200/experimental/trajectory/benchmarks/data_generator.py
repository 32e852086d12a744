"""Synthetic trajectories for store benchmarks (tunix/experimental/trajectory/benchmarks/data_generator.py:9-89).

A workload is a list of cumulative store sizes ("stages": write up to 100 trajectories, check recovery, write up to
1000, check again, ...) plus the shape of one trajectory. Trajectories are generated lazily and numbered from 1;
`trajectory_id_of(i)` is the id of the i-th, so a reader can ask for exactly the ones a stage should hold.

Payloads are not one constant string: the message of step s of trajectory t starts with a tag that names both, so a
store that mixes up steps or trajectories is caught by `expected_message`, while the bulk of the payload is shared
and costs no generation time.
"""
from __future__ import annotations

import dataclasses
from typing import Iterator, List, Sequence, Tuple

from .. import trajectory as trajectory_lib


@dataclasses.dataclass(frozen=True, kw_only=True)
class WorkloadConfig:
  cumulative_trajectory_checkpoints: Sequence[int] = (100, 1000, 10000)   # store size after each stage
  steps_per_trajectory: int = 20
  step_payload_chars: int = 20000                                          # ~20 KB per step

  def __post_init__(self) -> None:
    sizes = list(self.cumulative_trajectory_checkpoints)
    if not sizes:
      raise ValueError("cumulative_trajectory_checkpoints cannot be empty.")
    if any(int(s) != s or s <= 0 for s in sizes):
      raise ValueError(f"All checkpoints must be positive integers, got {sizes}")
    if any(b <= a for a, b in zip(sizes, sizes[1:])):
      raise ValueError(f"cumulative_trajectory_checkpoints must be strictly increasing, got {sizes}")
    if self.steps_per_trajectory <= 0:
      raise ValueError("steps_per_trajectory must be > 0.")
    if self.step_payload_chars <= 0:
      raise ValueError("step_payload_chars must be > 0.")

  @property
  def total_trajectories(self) -> int:
    return int(self.cumulative_trajectory_checkpoints[-1])


def trajectory_id_of(index: int) -> str:
  return f"traj_{index:06d}"


def expected_message(workload: WorkloadConfig, trajectory_index: int, step_id: int) -> str:
  tag = f"[{trajectory_index}:{step_id}]"
  return (tag + "x" * workload.step_payload_chars)[:max(workload.step_payload_chars, len(tag))]


def generate_trajectories(workload: WorkloadConfig, first: int = 1
                          ) -> Iterator[Tuple[trajectory_lib.TrajectoryMetadata, List[trajectory_lib.Step]]]:
  """(metadata, steps) of trajectories `first` .. the last stage's size."""
  agent = trajectory_lib.Agent(name="benchmark_agent", version="1.0")
  for index in range(first, workload.total_trajectories + 1):
    steps = [trajectory_lib.Step(step_id=s, source=trajectory_lib.Source.USER, message=expected_message(workload, index, s))
             for s in range(1, workload.steps_per_trajectory + 1)]
    yield trajectory_lib.TrajectoryMetadata(trajectory_id=trajectory_id_of(index), agent=agent), steps
