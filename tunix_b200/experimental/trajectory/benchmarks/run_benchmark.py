"""Command line of the trajectory-store recovery benchmark
(tunix/experimental/trajectory/benchmarks/run_benchmark.py:17-162).

  python -m tunix_b200.experimental.trajectory.benchmarks.run_benchmark \\
      --store file --root_dir /tmp/traj_bench --checkpoints 100,1000 --steps 20 --payload_chars 20000

`--store memory` measures the in-process store (a floor for the numbers); `--store file` the directory-backed one
with its asynchronous writer. The table printed at the end has one row per stage; `--json`
prints the same as one JSON object for scripts. Exit code 1 when a stage failed verification.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import shutil
import sys
import tempfile
from typing import List, Optional, Sequence, Tuple

from .. import async_writer, file_store, in_memory_store, store
from . import benchmark_lib, data_generator


@dataclasses.dataclass(frozen=True, kw_only=True)
class FileTrajectoryStoreConfig:
  root_dir: Optional[str] = None          # a fresh temporary directory (removed afterwards) when None

  def build(self) -> Tuple[store.TrajectoryReader, store.TrajectoryWriter, Optional[str]]:
    root, temporary = (self.root_dir, None) if self.root_dir else (tempfile.mkdtemp(prefix="traj_bench_"),) * 2
    st = file_store.FileTrajectoryStore(root, writer=async_writer.AsyncFileWriter())
    return st, st, temporary


@dataclasses.dataclass(frozen=True, kw_only=True)
class InMemoryTrajectoryStoreConfig:

  def build(self) -> Tuple[store.TrajectoryReader, store.TrajectoryWriter, Optional[str]]:
    st = in_memory_store.InMemoryTrajectoryStore()
    return st, st, None


@dataclasses.dataclass(frozen=True, kw_only=True)
class BenchmarkConfig:
  store: object = dataclasses.field(default_factory=InMemoryTrajectoryStoreConfig)
  workload: data_generator.WorkloadConfig = dataclasses.field(default_factory=data_generator.WorkloadConfig)
  as_json: bool = False


_COLUMNS = (("total", "total_trajectories", "{:,d}"), ("new", "checkpoint_write_count", "{:,d}"),
            ("write s", "write_duration_sec", "{:.3f}"), ("steps/s", "write_qps", "{:,.0f}"),
            ("MB/s", "write_mb_per_sec", "{:,.1f}"), ("scan ms", "metadata_scan_latency_ms", "{:,.1f}"),
            ("load ms", "trajectory_load_latency_ms", "{:,.1f}"), ("ok", "validation_passed", "{}"))


def format_report(report: benchmark_lib.BenchmarkReport) -> str:
  rows: List[List[str]] = [[title for title, _, _ in _COLUMNS]]
  for c in report.checkpoints:
    rows.append([fmt.format(getattr(c, field)) for _, field, fmt in _COLUMNS])
  widths = [max(len(r[i]) for r in rows) for i in range(len(_COLUMNS))]
  lines = [f"{report.writer_type} / {report.reader_type}: {report.workload.steps_per_trajectory} steps x "
           f"{report.workload.step_payload_chars:,d} chars per trajectory"]
  for n, row in enumerate(rows):
    lines.append("  ".join(cell.rjust(w) for cell, w in zip(row, widths)))
    if n == 0:
      lines.append("  ".join("-" * w for w in widths))
  lines += [f"stage {c.total_trajectories:,d}: {c.validation_error}" for c in report.checkpoints if c.validation_error]
  return "\n".join(lines)


def main(config: BenchmarkConfig) -> benchmark_lib.BenchmarkReport:
  reader, writer, temporary = config.store.build()
  try:
    report = benchmark_lib.run_recovery_benchmark(reader, writer, config.workload,
                                                  progress=None if config.as_json else print)
  finally:
    close = getattr(writer, "close", None)
    if callable(close):
      close()
    if temporary:
      shutil.rmtree(temporary, ignore_errors=True)
  if config.as_json:
    print(json.dumps({"reader": report.reader_type, "writer": report.writer_type,
                      "workload": dataclasses.asdict(report.workload),
                      "checkpoints": [dataclasses.asdict(c) for c in report.checkpoints]}))
  else:
    print(format_report(report))
  return report


def parse_args(argv: Sequence[str]) -> BenchmarkConfig:
  p = argparse.ArgumentParser(description="Recovery benchmark of a trajectory store")
  p.add_argument("--store", choices=("memory", "file"), default="memory")
  p.add_argument("--root_dir", default=None)
  p.add_argument("--checkpoints", default="100,1000", help="cumulative store sizes, comma separated")
  p.add_argument("--steps", type=int, default=20)
  p.add_argument("--payload_chars", type=int, default=20000)
  p.add_argument("--json", action="store_true")
  a = p.parse_args(list(argv))
  st = (FileTrajectoryStoreConfig(root_dir=a.root_dir) if a.store == "file"
        else InMemoryTrajectoryStoreConfig())
  workload = data_generator.WorkloadConfig(cumulative_trajectory_checkpoints=[int(x) for x in a.checkpoints.split(",") if x],
                                           steps_per_trajectory=a.steps, step_payload_chars=a.payload_chars)
  return BenchmarkConfig(store=st, workload=workload, as_json=a.json)


if __name__ == "__main__":
  sys.exit(0 if main(parse_args(sys.argv[1:])).passed else 1)
