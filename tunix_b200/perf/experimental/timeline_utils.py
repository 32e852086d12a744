"""Timeline ids and post-processing (tunix/perf/experimental/timeline_utils.py)."""
from __future__ import annotations

import threading
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np

from . import timeline
from . import constants


def generate_host_timeline_id() -> str:
  return f"host-{threading.get_ident()}"


def is_host_timeline(tl_id: str) -> bool:
  return tl_id.startswith("host-")


def generate_queued_timeline_id(tl_id: str) -> str:
  return f"{tl_id}_queue"


def is_queued_timeline(tl_id: str) -> bool:
  return tl_id.endswith("_queue")


def generate_device_timeline_id(device_id: Any) -> str:
  """"cuda3" for torch.device('cuda', 3) or rank 3; strings pass through."""
  if isinstance(device_id, str):
    return device_id
  if isinstance(device_id, (int, np.integer)):
    return f"cuda{int(device_id)}"
  t, i = getattr(device_id, "type", None), getattr(device_id, "index", None)
  if t is not None:
    return f"{t}{0 if i is None else i}"
  if hasattr(device_id, "platform") and hasattr(device_id, "id"):
    return f"{device_id.platform}{device_id.id}"
  raise ValueError(f"Unsupported device id type: {type(device_id)}")


def generate_device_timeline_ids(devices: Optional[Sequence[Any]]) -> List[str]:
  if devices is None:
    return []
  if isinstance(devices, np.ndarray):
    devices = devices.flatten().tolist()
  return [generate_device_timeline_id(d) for d in devices]


def is_timeline_only_of_allowed_type(tl: timeline.Timeline, allowed_span_names: Sequence[str],
                                     include_cur_step: bool = False) -> bool:
  steps = tl.all_steps if include_cur_step else tl.committed_steps
  return all(sp.name in allowed_span_names for step in steps for sp in step.values())


def sequentialize_overlapping_spans(
    spans_dict: Mapping[int, timeline.Span]) -> Tuple[Dict[int, timeline.Span], Dict[int, timeline.Span]]:
  """A device runs one thing at a time: of overlapping spans the earlier one is active and the
  later one starts when it ends; the wait in front becomes a "queue" span. A span whose whole
  duration lies inside the wait is only queued. Returns (active, queue), both keyed by span id."""
  active: Dict[int, timeline.Span] = {}
  queue: Dict[int, timeline.Span] = {}
  busy_until = float("-inf")
  for sid, sp in sorted(spans_dict.items(), key=lambda kv: (kv[1].begin, kv[1].end)):
    if not sp.ended:
      active[sid] = sp
      continue
    if sp.begin >= busy_until:
      active[sid] = sp
      busy_until = sp.end
      continue
    wait_end = min(busy_until, sp.end)
    q = timeline.Span(name=sp.name, begin=sp.begin, id=sid, parent_id=sp.parent_id,
                      tags={**(sp.tags or {}), constants.QUEUE: True})
    q.end = wait_end
    queue[sid] = q
    if sp.end > busy_until:
      a = timeline.Span(name=sp.name, begin=busy_until, id=sid, parent_id=sp.parent_id, tags=sp.tags)
      a.end = sp.end
      active[sid] = a
      busy_until = sp.end
  return active, queue
