"""Turns the span trees of one global RL step into `perf/*` metrics
(tunix/perf/export.py:53-569).

Emitted per global step: `perf/global_step_time`, `perf/weight_sync_time`, and `sum` / `mean` of
`rollout_time`, `refer_inference_time`, `actor_train_time`, `actor_train_step_time`. When the
rollout runs on ranks of its own (role meshes differ) `perf/rollout_idle_time`,
`perf/first_micro_batch_rollout_time` and the gaps between rollout micro-batches are added; a
fully disaggregated layout adds the reference / actor idle and gap analogues.

Spans are looked up by name in every host-thread timeline and attributed to the last
`global_step` group of the main thread by time overlap, so the producer thread's `rollout` and
`refer_inference` spans are found even though they are not nested under the main thread's group.
"""
from __future__ import annotations

import logging
from functools import partial
from typing import Any, Callable, Dict, List, Optional, Tuple

import numpy as np

from . import trace
from .metrics import MetricsT, PerfSpanQuery
from .perfetto import PerfettoTraceWriter
from .span import Span, SpanGroup

log = logging.getLogger(__name__)
MetricsExportFn = Callable[[PerfSpanQuery], MetricsT]


def _mean(x: List[float]) -> float:
  return float(np.mean(x)) if x else 0.0


def _gaps(spans: List[Span]) -> List[float]:
  s = sorted(spans, key=lambda x: x.begin)
  return [max(0.0, b.begin - a.end) for a, b in zip(s[:-1], s[1:])]


class PerfMetricsExport:
  """Factories for export functions."""

  @staticmethod
  def from_role_to_devices(role_to_devices: Dict[str, List[str]], trace_writer: Optional[PerfettoTraceWriter] = None,
                           log_rollout_time_at_micro_batch_level: bool = False,
                           log_actor_train_time_at_micro_batch_level: bool = False) -> MetricsExportFn:
    r2d = role_to_devices
    if r2d["rollout"] == r2d["actor"] == r2d["refer"]:
      layout = "colocated"
    elif r2d["rollout"] != r2d["actor"] and r2d["actor"] == r2d["refer"]:
      layout = "rollout_split"
    elif r2d["rollout"] != r2d["actor"] and r2d["actor"] != r2d["refer"]:
      layout = "fully_disaggregated"
    else:
      raise ValueError("Unsupported mesh configuration.")
    log.info("Collecting perf metrics for layout: %s", layout)
    return partial(PerfMetricsExport._grpo_metrics, layout, trace_writer, log_rollout_time_at_micro_batch_level,
                   log_actor_train_time_at_micro_batch_level)

  @staticmethod
  def from_cluster_config(cluster_config: Any, log_rollout_time_at_micro_batch_level: bool = False,
                          log_actor_train_time_at_micro_batch_level: bool = False) -> MetricsExportFn:
    from ..common.datatypes import Role

    def devs(role):
      m = cluster_config.role_to_mesh.get(role)
      return [trace.create_device_timeline_id(r) for r in (m.ranks() if m is not None else [0])]
    opts = cluster_config.training_config.perf_metrics_options
    writer = PerfettoTraceWriter(opts.trace_dir) if (opts is not None and opts.enable_trace_writer) else None
    refer = devs(Role.REFERENCE) if Role.REFERENCE in cluster_config.role_to_mesh else devs(Role.ACTOR)
    return PerfMetricsExport.from_role_to_devices(
        {"rollout": devs(Role.ROLLOUT), "actor": devs(Role.ACTOR), "refer": refer}, writer,
        log_rollout_time_at_micro_batch_level, log_actor_train_time_at_micro_batch_level)

  create_metrics_export_fn = from_cluster_config

  @staticmethod
  def _collect(query: PerfSpanQuery):
    main = query().main().last_group("global_step").get()
    if not main:
      log.warning("global_step is None")
      return None
    gs = main[0]
    lo, hi = gs.begin, gs.end
    rollout, refer, trains, steps, sync = [], [], [], [], []
    for tid in query.get_timeline_ids():
      if not tid.startswith("thread-"):
        continue
      root = query().timeline(tid).get()[0]
      inside = lambda s: s.ended and s.end >= lo and s.begin <= hi
      rollout += [s for s in root.find_all_spans_recursive("rollout") if inside(s)]
      refer += [s for s in root.find_all_spans_recursive("refer_inference") if inside(s)]
      trains += [g for g in root.find_all_groups_recursive("actor_training") if inside(g)]
      steps += [s for s in root.find_all_spans_recursive("peft_train_step") if inside(s)]
      sync += [s for s in root.find_all_spans_recursive("weight_sync") if inside(s)]
    return gs, rollout, refer, trains, steps, sync

  @staticmethod
  def _grpo_metrics(layout: str, trace_writer, log_rollout: bool, log_train: bool, query: PerfSpanQuery) -> MetricsT:
    got = PerfMetricsExport._collect(query)
    if got is None:
      return {}
    gs, rollout, refer, trains, steps, sync = got
    if sync:
      ws = sync[-1]
    else:
      ws = Span("weight_sync", gs.end)
      ws.end = gs.end
    rt = [s.duration for s in rollout]
    ft = [s.duration for s in refer]
    tt = [g.duration for g in trains]
    st = [s.duration for s in steps]
    if log_rollout:
      for i, t in enumerate(rt):
        log.info("rollout time [%s] = %s sec", i, t)
    if log_train:
      for i, t in enumerate(tt):
        log.info("actor train time [%s] = %s sec", i, t)
    if trace_writer is not None:
      trace_writer.log_trace([gs], rollout, refer, trains)
    m: MetricsT = {
        "perf/global_step_time": (gs.duration, None),
        "perf/weight_sync_time": (ws.duration, None),
        "perf/sum/rollout_time": (float(np.sum(rt)) if rt else 0.0, None),
        "perf/sum/refer_inference_time": (float(np.sum(ft)) if ft else 0.0, None),
        "perf/sum/actor_train_time": (float(np.sum(tt)) if tt else 0.0, None),
        "perf/sum/actor_train_step_time": (float(np.sum(st)) if st else 0.0, None),
        "perf/mean/rollout_time": (_mean(rt), None),
        "perf/mean/refer_inference_time": (_mean(ft), None),
        "perf/mean/actor_train_time": (_mean(tt), None),
        "perf/mean/actor_train_step_time": (_mean(st), None),
    }
    if layout in ("rollout_split", "fully_disaggregated") and rollout:
      last_end = max(s.end for s in rollout)
      g = _gaps(rollout)
      m["perf/rollout_idle_time"] = (max(0.0, ws.begin - last_end), None)
      m["perf/first_micro_batch_rollout_time"] = (sorted(rollout, key=lambda s: s.begin)[0].duration, None)
      m["perf/sum/between_micro_batch_gap_time"] = (float(np.sum(g)) if g else 0.0, None)
      m["perf/mean/between_micro_batch_gap_time"] = (_mean(g), None)
    if layout == "fully_disaggregated":
      if refer:
        g = _gaps(refer)
        m["perf/refer_idle_time"] = (max(0.0, ws.begin - max(s.end for s in refer)), None)
        m["perf/sum/refer_gap_time"] = (float(np.sum(g)) if g else 0.0, None)
        m["perf/mean/refer_gap_time"] = (_mean(g), None)
      if trains:
        g = _gaps(trains)
        m["perf/actor_idle_time"] = (max(0.0, sorted(trains, key=lambda s: s.begin)[0].begin - gs.begin), None)
        m["perf/sum/actor_gap_time"] = (float(np.sum(g)) if g else 0.0, None)
        m["perf/mean/actor_gap_time"] = (_mean(g), None)
    return m
