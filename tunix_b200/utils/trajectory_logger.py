"""CSV logging of trajectories, synchronous and on a background thread
(tunix/utils/trajectory_logger.py:31-250).

One row per item; nested values are stored as JSON text in their cell. The file is named after
the dataclass of the item (`trajectory_log` for dicts) plus an optional suffix. New keys that
appear later are appended as new columns by rewriting the header.
"""
from __future__ import annotations

import atexit
import csv
import dataclasses
import json
import logging
import os
import queue
import threading
import time
from typing import Any, Dict, List, Optional

import numpy as np


def _make_serializable(item: Any) -> Any:
  if isinstance(item, dict):
    return {str(k): _make_serializable(v) for k, v in item.items()}
  if isinstance(item, (list, tuple)):
    return [_make_serializable(v) for v in item]
  if dataclasses.is_dataclass(item) and not isinstance(item, type):
    return _make_serializable(dataclasses.asdict(item))
  if isinstance(item, np.ndarray):
    return item.tolist()
  if isinstance(item, np.generic):
    return item.item()
  if hasattr(item, "detach") and hasattr(item, "cpu"):
    return item.detach().cpu().tolist()
  if isinstance(item, (float, int, bool, str)) or item is None:
    return item
  if hasattr(item, "name") and hasattr(item, "value"):     # enums
    return item.name
  return str(item)


def _item_name(item: Any) -> Optional[str]:
  return item.__class__.__name__ if dataclasses.is_dataclass(item) and not isinstance(item, type) else None


def _cell(v: Any) -> Any:
  return json.dumps(v) if isinstance(v, (dict, list)) else v


def log_item(log_path: str, item: Any, suffix: Optional[str] = None) -> Optional[str]:
  """Appends `item` (dataclass, dict, or list of those) to a CSV under `log_path`; returns the file."""
  if log_path is None:
    raise ValueError("No directory for logging provided.")
  if isinstance(item, list) and not item:
    logging.warning("Trying to log an empty list, skipping.")
    return None
  if not (isinstance(item, (dict, list)) or _item_name(item)):
    raise ValueError(f"Item {item} is not a dataclass, dictionary or list.")
  rows = _make_serializable(item if isinstance(item, list) else [item])
  os.makedirs(log_path, exist_ok=True)
  stem = _item_name(item[0] if isinstance(item, list) else item) or "trajectory_log"
  path = os.path.join(log_path, f"{stem}_{suffix}.csv" if suffix else f"{stem}.csv")
  old_rows: List[Dict[str, Any]] = []
  header: List[str] = []
  if os.path.exists(path):
    with open(path, newline="") as f:
      rd = csv.DictReader(f)
      header = list(rd.fieldnames or [])
      new_keys = [k for r in rows for k in r if k not in header]
      if new_keys:
        old_rows = list(rd)
  cols = header + [k for k in dict.fromkeys(k for r in rows for k in r) if k not in header]
  if old_rows or not header:
    tmp = path + ".tmp"
    with open(tmp, "w", newline="") as f:
      wr = csv.DictWriter(f, fieldnames=cols)
      wr.writeheader()
      wr.writerows(old_rows)
      wr.writerows({k: _cell(v) for k, v in r.items()} for r in rows)
    os.replace(tmp, path)
  else:
    with open(path, "a", newline="") as f:
      csv.DictWriter(f, fieldnames=cols).writerows({k: _cell(v) for k, v in r.items()} for r in rows)
  return path


class AsyncTrajectoryLogger:
  """Queues items and writes them from one background thread, batching whatever has piled up."""

  def __init__(self, log_dir: str):
    self._log_dir = log_dir
    self._suffix = str(int(time.time()))
    self._q: "queue.Queue" = queue.Queue()
    self._stopped = False
    self._thread = threading.Thread(target=self._work, daemon=True, name="trajectory-logger")
    self._thread.start()
    atexit.register(self.stop)

  def _work(self) -> None:
    while True:
      item = self._q.get()
      if item is None:
        self._q.task_done()
        return
      items, stop = [item], False
      while True:
        try:
          nxt = self._q.get_nowait()
        except queue.Empty:
          break
        if nxt is None:
          stop = True
          break
        items.append(nxt)
      try:
        log_item(self._log_dir, items, self._suffix)
      except Exception:
        logging.exception("Failed to log trajectories.")
      finally:
        for _ in range(len(items) + (1 if stop else 0)):
          self._q.task_done()
      if stop:
        return

  def log_item_async(self, item: Any) -> None:
    if self._stopped:
      logging.warning("trajectory logger already stopped; item dropped")
      return
    self._q.put(item)

  def flush(self) -> None:
    self._q.join()

  def stop(self) -> None:
    if self._stopped:
      return
    self._stopped = True
    self._q.put(None)
    self._thread.join(timeout=30)
