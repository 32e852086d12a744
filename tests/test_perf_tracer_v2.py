"""The tag-based tracer: host lanes per thread, device lanes closed by the completion of the issued work, several
devices per span, nesting on the host against flat device lanes, queue lanes for work that waited, step commits,
export, waiting for stragglers, failures inside waits, and the no-op tracer."""
import threading
import time

import numpy as np
import pytest

from tunix_b200.perf import experimental as pv2
from tunix_b200.perf.experimental import timeline_utils
from tunix_b200.perf.experimental.timeline import Span, Timeline


class Work:
  """Something a span can wait on: finishes `seconds` after it was created, on a timer thread."""

  def __init__(self, seconds, fail=False):
    self.done, self.fail = threading.Event(), fail
    threading.Timer(seconds, self.done.set).start()

  def wait(self):
    self.done.wait(5)
    if self.fail:
      raise RuntimeError("device fell off the bus")


def lanes(tracer):
  return tracer._get_timelines()


def names(lane, step=-1, committed=True):
  steps = lane.committed_steps if committed else lane.all_steps
  return [s.name for s in steps[step].values()]


def test_a_tracer_without_devices_records_the_host_only():
  tr = pv2.PerfTracer()
  assert list(tr.all_devices) == []
  with tr.span("load", tags={"step": 1}):
    time.sleep(0.01)
  tr.process_and_commit_timelines()
  (host,) = lanes(tr).values()
  (span,) = host.committed_steps[0].values()
  assert span.name == "load" and span.tags == {"step": 1} and span.duration >= 0.01 and span.ended


def test_device_spans_end_when_the_issued_work_ends_not_when_the_host_block_does():
  tr = pv2.PerfTracer(devices=["gpu0", "gpu1"])
  assert len(tr.all_devices) == 2
  with tr.span("rollout", devices=["gpu0", "gpu1"], tags={"role": "actor"}) as pending:
    pending.async_end([Work(0.08)])
  t_host_done = time.perf_counter()
  tr.synchronize()
  waited = time.perf_counter() - t_host_done
  assert waited >= 0.04                                           # synchronize waited for the stragglers
  tr.process_and_commit_timelines()
  host = lanes(tr)[timeline_utils.generate_host_timeline_id()]
  (h,) = host.committed_steps[0].values()
  for dev in tr.all_devices:
    (d,) = lanes(tr)[dev].committed_steps[0].values()
    assert d.name == "rollout" and d.tags == {"role": "actor"}
    assert d.begin == pytest.approx(h.begin) and d.duration >= 0.07 > h.duration      # same start, later end


def test_devices_may_be_arrays_and_one_device_can_stand_for_a_mesh():
  grid = np.array([["a", "b"], ["c", "d"]])
  tr = pv2.PerfTracer(devices=grid)
  with tr.span("step", devices=grid) as pending:
    pending.async_end(None)
  tr.process_and_commit_timelines()
  assert sum(bool(lanes(tr)[d].committed_steps[0]) for d in tr.all_devices) == 4
  first_only = pv2.PerfTracer(devices=grid, collect_on_first_device_per_mesh=True)
  with first_only.span("step", devices=grid):
    pass
  first_only.process_and_commit_timelines()
  used = [d for d in first_only.all_devices if first_only._get_timelines()[d].committed_steps[0]]
  assert len(used) == 1 and used[0] == timeline_utils.generate_device_timeline_id("a")


def test_host_spans_nest_while_device_lanes_stay_flat():
  tr = pv2.PerfTracer(devices=["gpu0"], concurrent_spans="all")       # keep both on the lane: nothing is re-sequenced
  with tr.span("outer", devices=["gpu0"]) as outer:
    with tr.span("inner", devices=["gpu0"]) as inner:
      inner.async_end(None)
    outer.async_end(None)
  tr.process_and_commit_timelines()
  host = lanes(tr)[timeline_utils.generate_host_timeline_id()]
  by_name = {s.name: s for s in host.committed_steps[0].values()}
  assert by_name["inner"].parent_id == by_name["outer"].id and by_name["outer"].parent_id is None
  dev = lanes(tr)[tr.all_devices[0]]
  assert sorted(names(dev)) == ["inner", "outer"] and all(s.parent_id is None for s in dev.committed_steps[0].values())


def test_every_thread_gets_its_own_host_lane():
  tr = pv2.PerfTracer()

  def worker(k):
    with tr.span(f"t{k}"):
      time.sleep(0.01)
  threads = [threading.Thread(target=worker, args=(k,)) for k in range(3)]
  for t in threads: t.start()
  for t in threads: t.join()
  with tr.span("main"):
    pass
  tr.process_and_commit_timelines()
  recorded = sorted(n for lane in lanes(tr).values() for step in lane.committed_steps for n in (s.name for s in step.values()))
  assert recorded == ["main", "t0", "t1", "t2"]
  assert len([l for l in lanes(tr).values() if l.committed_steps and l.committed_steps[0]]) == 4       # no lane is shared


def test_work_that_waited_behind_other_work_moves_to_a_queue_lane_unless_declared_concurrent():
  def run(**kw):
    tr = pv2.PerfTracer(devices=["gpu0"], **kw)
    with tr.span("first", devices=["gpu0"]) as p:
      p.async_end([Work(0.06)])
    with tr.span("second", devices=["gpu0"]) as p:
      p.async_end([Work(0.1)])
    tr.process_and_commit_timelines()
    return tr
  tr = run()
  dev_id = tr.all_devices[0]
  dev = lanes(tr)[dev_id]
  spans = {s.name: s for s in dev.committed_steps[0].values()}
  assert spans["second"].begin == pytest.approx(spans["first"].end)              # no overlap is left on the device
  queue = lanes(tr)[timeline_utils.generate_queued_timeline_id(dev_id)]
  (q,) = queue.committed_steps[0].values()
  assert q.name == "second" and q.end == pytest.approx(spans["first"].end) and q.begin < q.end
  for declared in (["second"], "all"):
    tr = run(concurrent_spans=declared)
    assert timeline_utils.generate_queued_timeline_id(tr.all_devices[0]) not in lanes(tr)
    spans = {s.name: s for s in lanes(tr)[tr.all_devices[0]].committed_steps[0].values()}
    assert spans["second"].begin < spans["first"].end                            # they really overlapped


def test_steps_are_committed_one_by_one_and_exported():
  seen = []
  tr = pv2.PerfTracer(devices=["gpu0"], export_fn=lambda timelines: (seen.append(timelines), {"n": (len(timelines), None)})[1])
  for step in range(2):
    with tr.span("train", devices=["gpu0"], tags={"step": step}) as p:
      p.async_end(None)
    assert tr.export() == {"n": (2, None)}
  dev = seen[-1][tr.all_devices[0]]
  assert [list(s.tags.values()) for step in dev.committed_steps for s in step.values()] == [[0], [1]]
  assert dev.cur_step == {} and pv2.PerfTracer().export() == {}


def test_a_failing_wait_loses_its_span_only(caplog):
  tr = pv2.PerfTracer(devices=["gpu0"])
  with caplog.at_level("ERROR"):
    with tr.span("doomed", devices=["gpu0"]) as p:
      p.async_end([Work(0.01, fail=True)])
    with tr.span("fine", devices=["gpu0"]) as p:
      p.async_end([Work(0.01)])
    tr.process_and_commit_timelines()
  assert "doomed" in caplog.text and names(lanes(tr)[tr.all_devices[0]]) == ["fine"]


def test_timeline_rules():
  tl = Timeline("lane", 10.0)
  a = tl.start_span("a", 11.0)
  tl.stop_span(12.0)
  assert a.duration == 1.0 and a.ended and tl.cur_step == {a.id: a}
  with pytest.raises(ValueError, match="no more spans"):
    tl.stop_span(13.0)
  open_span = tl.start_span("never closed", 13.0)
  assert not open_span.ended
  tl.commit_step()
  assert names(tl) == ["a"] and tl.all_steps[-1] == {}                # unfinished work does not reach a committed step
  s = Span(name="x", begin=5.0, id=0)
  s.add_tag("k", 1)
  assert s.tags == {"k": 1} and "lane" in repr(tl)
  tr = pv2.PerfTracer(devices=["gpu0"])
  tr.print()                                                          # waits, then prints every lane; must not raise


def test_the_noop_tracer_accepts_everything_and_records_nothing():
  noop = pv2.NoopTracer()
  with noop.span("x", devices=["gpu0"], tags={"a": 1}) as p:
    p.async_end([Work(0.0)])
  noop.synchronize(); noop.print()
  assert noop.export() == {} and list(noop.all_devices) == []
