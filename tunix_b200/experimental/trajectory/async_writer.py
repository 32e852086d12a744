"""Background writer that turns trajectory steps into files.

One daemon thread drains a FIFO queue, so steps of a trajectory reach the disk
in the order they were logged without per-file locks. The thread starts on the
first write (a read-only store never spawns it). Every file is written to a
temporary name and renamed, so a reader never sees half a file. I/O errors are
logged and swallowed: trajectory logs are diagnostics and must not stop a
training job. ``flush`` returns once everything queued before it is on disk.

Contract of tunix/experimental/trajectory/async_writer.py.
"""

from __future__ import annotations

import dataclasses
import logging
import os
import queue
import threading

import pydantic

log = logging.getLogger(__name__)


def _dump_json(model: pydantic.BaseModel) -> str:
  return model.model_dump_json(exclude_none=True, indent=2)


def atomic_write_text(path: str, text: str) -> None:
  tmp = f"{path}.tmp.{os.getpid()}.{threading.get_ident()}"
  with open(tmp, "w", encoding="utf-8") as f:
    f.write(text)
  os.replace(tmp, path)


@dataclasses.dataclass
class _WriteTask:
  trajectory_id: str
  trajectory_dir: str
  metadata_path: str
  metadata_json: str
  step_path: str | None = None
  step_json: str | None = None


class AsyncFileWriter:

  def __init__(self) -> None:
    self._queue: queue.Queue[_WriteTask | None] = queue.Queue()
    self._metadata_hash: dict[str, int] = {}
    self._lock = threading.Lock()
    self._thread: threading.Thread | None = None
    self._closed = False
    self.errors = 0

  def _enqueue(self, task: _WriteTask) -> None:
    """Starts the worker on first use and queues the task, in one critical section with `close`: a task is
    either refused or lands before the shutdown marker, never behind it (where nothing would ever write it and
    `flush` would wait forever)."""
    with self._lock:
      if self._closed:
        raise RuntimeError("AsyncFileWriter is closed")
      if self._thread is None or not self._thread.is_alive():
        self._thread = threading.Thread(
            target=self._worker_loop, name="trajectory-writer", daemon=True)
        self._thread.start()
      self._queue.put(task)

  def write_step(self, *, trajectory_id: str, trajectory_dir: str,
                 metadata_path: str, metadata: pydantic.BaseModel,
                 step_path: str | None = None,
                 step: pydantic.BaseModel | None = None) -> None:
    """Queues a metadata write and, when given, a step write.

    Serialisation happens here, on the caller's thread, which is the snapshot:
    later changes to `metadata` or `step` do not reach the file.
    """
    self._enqueue(_WriteTask(
        trajectory_id=trajectory_id, trajectory_dir=trajectory_dir,
        metadata_path=metadata_path, metadata_json=_dump_json(metadata),
        step_path=step_path,
        step_json=None if step is None else _dump_json(step)))

  def _worker_loop(self) -> None:
    while True:
      task = self._queue.get()
      try:
        if task is None:
          return
        self._process_task(task)
      except Exception:  # pylint: disable=broad-exception-caught
        self.errors += 1
        log.exception("trajectory write failed")
      finally:
        self._queue.task_done()

  def _process_task(self, task: _WriteTask) -> None:
    os.makedirs(task.trajectory_dir, exist_ok=True)
    h = hash(task.metadata_json)
    if self._metadata_hash.get(task.trajectory_id) != h:
      atomic_write_text(task.metadata_path, task.metadata_json)
      self._metadata_hash[task.trajectory_id] = h
    if task.step_path is not None and task.step_json is not None:
      atomic_write_text(task.step_path, task.step_json)

  def flush(self) -> None:
    if self._thread is not None:
      self._queue.join()

  def close(self, timeout: float | None = 5.0) -> None:
    with self._lock:
      if self._closed:
        return
      self._closed = True
      thread = self._thread
      if thread is not None and thread.is_alive():
        self._queue.put(None)
    if thread is not None and thread.is_alive():
      thread.join(timeout)
      if thread.is_alive():
        log.warning("trajectory writer did not finish within %s s; %d task(s) may be unwritten", timeout,
                    self._queue.qsize())

  def __del__(self) -> None:
    try:
      self.close(timeout=1.0)
    except Exception:  # pylint: disable=broad-exception-caught
      pass
