"""Recovery benchmark of a trajectory store (tunix/experimental/trajectory/benchmarks/benchmark_lib.py:13-241).

What a restarted RL job does with its trajectory store is: list every trajectory's metadata, then load the ones it
still needs. How long that takes depends on how much the store already holds, so the benchmark grows the store in
stages and, after each, times exactly those two calls next to the write throughput that filled the stage:

    stage k:  add_step x (new trajectories x steps) -> flush      [steps/s, MB/s]
              get_trajectories_metadata()                         [ms]
              get_trajectories(all ids so far)                    [ms]
              verify: counts, and on a sample the step count and each step's payload

The verification is part of the result (`validation_passed`, `validation_error`), not an exception: a store that
loses data under load should show up in the report of the stage where it happened.
"""
from __future__ import annotations

import dataclasses
import time
from typing import Callable, Iterator, List, Optional

from .. import store
from . import data_generator


class Timer:
  """`with Timer() as t: ...` then `t.duration_sec` / `t.duration_ms`; reusable."""

  def __init__(self) -> None:
    self.start = 0.0
    self.duration_sec = 0.0

  def __enter__(self) -> "Timer":
    self.duration_sec = 0.0
    self.start = time.perf_counter()
    return self

  def __exit__(self, *exc: object) -> None:
    self.duration_sec = time.perf_counter() - self.start

  @property
  def duration_ms(self) -> float:
    return self.duration_sec * 1e3


def _rate(amount: float, seconds: float) -> float:
  return amount / seconds if seconds > 0 else float("inf")


@dataclasses.dataclass(frozen=True, kw_only=True)
class BenchmarkCheckpointMetrics:
  checkpoint_write_count: int          # trajectories written in this stage
  total_trajectories: int              # store size after it
  write_duration_sec: float            # add_step calls + flush
  write_qps: float                     # steps per second
  write_mb_per_sec: float              # message bytes per second / 2**20
  metadata_scan_latency_ms: float
  trajectory_load_latency_ms: float
  validation_passed: bool
  validation_error: Optional[str] = None


@dataclasses.dataclass(frozen=True, kw_only=True)
class BenchmarkReport:
  reader_type: str
  writer_type: str
  workload: data_generator.WorkloadConfig
  checkpoints: List[BenchmarkCheckpointMetrics]

  @property
  def passed(self) -> bool:
    return all(c.validation_passed for c in self.checkpoints)


def _verify(workload: data_generator.WorkloadConfig, size: int, metadata: list, loaded: list, sample: int) -> Optional[str]:
  if len(metadata) != size:
    return f"Expected {size} metadata entries, got {len(metadata)}"
  if len(loaded) != size:
    return f"Expected {size} loaded trajectories, got {len(loaded)}"
  stride = max(1, size // max(1, sample))
  for index in list(range(1, size + 1, stride)) + [size]:
    traj = loaded[index - 1]
    if traj.trajectory_id != data_generator.trajectory_id_of(index):
      return f"Position {index} holds {traj.trajectory_id!r}, expected {data_generator.trajectory_id_of(index)!r}"
    if len(traj.steps) != workload.steps_per_trajectory:
      return f"{traj.trajectory_id} has {len(traj.steps)} steps, expected {workload.steps_per_trajectory}"
    for step in traj.steps:
      if step.message != data_generator.expected_message(workload, index, step.step_id):
        return f"{traj.trajectory_id} step {step.step_id} came back with a different payload"
  return None


def _run_checkpoint(reader: store.TrajectoryReader, writer: store.TrajectoryWriter, data_iter: Iterator,
                    workload: data_generator.WorkloadConfig, current: int, target: int, sample: int,
                    say: Callable[[str], None]) -> BenchmarkCheckpointMetrics:
  say(f"  writing trajectories {current + 1:,d}..{target:,d}")
  steps = payload_bytes = 0
  with Timer() as writing:
    for _ in range(target - current):
      metadata, traj_steps = next(data_iter)
      for step in traj_steps:
        writer.add_step(step, metadata)
        payload_bytes += len(step.message)
      steps += len(traj_steps)
    writer.flush()
  say(f"  recovering {target:,d} trajectories")
  with Timer() as scanning:
    metadata_list = reader.get_trajectories_metadata()
  ids = [data_generator.trajectory_id_of(i) for i in range(1, target + 1)]
  with Timer() as loading:
    try:
      loaded, load_error = reader.get_trajectories(ids), None
    except KeyError as e:                         # a trajectory the store lost
      loaded, load_error = [], f"get_trajectories failed: {e}"
  error = load_error or _verify(workload, target, metadata_list, loaded, sample)
  return BenchmarkCheckpointMetrics(
      checkpoint_write_count=target - current, total_trajectories=target, write_duration_sec=writing.duration_sec,
      write_qps=_rate(steps, writing.duration_sec), write_mb_per_sec=_rate(payload_bytes / 2**20, writing.duration_sec),
      metadata_scan_latency_ms=scanning.duration_ms, trajectory_load_latency_ms=loading.duration_ms,
      validation_passed=error is None, validation_error=error)


def run_recovery_benchmark(reader: store.TrajectoryReader, writer: store.TrajectoryWriter,
                           workload: data_generator.WorkloadConfig, *, verify_sample: int = 16,
                           progress: Optional[Callable[[str], None]] = print) -> BenchmarkReport:
  """Runs every stage of `workload` against the (initially empty) store behind `reader` / `writer`."""
  say = progress or (lambda _line: None)
  stages = list(workload.cumulative_trajectory_checkpoints)
  data_iter = data_generator.generate_trajectories(workload)
  results: List[BenchmarkCheckpointMetrics] = []
  current = 0
  for number, target in enumerate(stages, start=1):
    say(f"[{number}/{len(stages)}] stage up to {target:,d} trajectories")
    stage = _run_checkpoint(reader, writer, data_iter, workload, current, int(target), verify_sample, say)
    verdict = "ok" if stage.validation_passed else f"FAILED: {stage.validation_error}"
    say(f"[{number}/{len(stages)}] {stage.write_qps:,.1f} steps/s, {stage.write_mb_per_sec:,.2f} MB/s, "
        f"scan {stage.metadata_scan_latency_ms:,.1f} ms, load {stage.trajectory_load_latency_ms:,.1f} ms - {verdict}")
    results.append(stage)
    current = int(target)
  return BenchmarkReport(reader_type=type(reader).__name__, writer_type=type(writer).__name__, workload=workload,
                         checkpoints=results)
