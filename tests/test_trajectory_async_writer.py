"""The background trajectory writer: non-blocking queueing, FIFO order, snapshots at call time, lazy thread start,
metadata rewritten only when it changes, errors swallowed and counted, close semantics under concurrency."""
import json
import os
import threading
import time

import pydantic
import pytest

from tunix_b200.experimental.trajectory import async_writer as aw


class Meta(pydantic.BaseModel):
  trajectory_id: str
  note: str = ""
  tags: list = []


class Step(pydantic.BaseModel):
  step_id: int
  text: str = ""
  values: list = []


def paths(root, tid, step=None):
  d = os.path.join(root, tid)
  return dict(trajectory_id=tid, trajectory_dir=d, metadata_path=os.path.join(d, "metadata.json"),
              step_path=None if step is None else os.path.join(d, f"step_{step}.json"))


def read(path):
  with open(path) as f:
    return json.load(f)


def test_writes_return_at_once_and_flush_makes_them_durable(tmp_path):
  w = aw.AsyncFileWriter()
  slow = w._process_task

  def delayed(task):
    time.sleep(0.1)
    slow(task)
  w._process_task = delayed
  t0 = time.perf_counter()
  for k in range(3):
    w.write_step(**paths(str(tmp_path), "t1", k), metadata=Meta(trajectory_id="t1"), step=Step(step_id=k, text=f"s{k}"))
  assert time.perf_counter() - t0 < 0.09                          # three slow writes queued, none waited for
  w.flush()
  assert [read(tmp_path / "t1" / f"step_{k}.json")["text"] for k in range(3)] == ["s0", "s1", "s2"]
  assert read(tmp_path / "t1" / "metadata.json") == {"trajectory_id": "t1", "note": "", "tags": []}
  assert not [f for f in os.listdir(tmp_path / "t1") if ".tmp." in f]      # written under a temporary name, renamed
  w.close()


def test_metadata_only_writes_and_fifo_order_across_trajectories(tmp_path):
  w = aw.AsyncFileWriter()
  order = []
  real = w._process_task
  w._process_task = lambda task: (order.append((task.trajectory_id, task.step_path and os.path.basename(task.step_path))),
                                  real(task))[1]
  w.write_step(**paths(str(tmp_path), "a"), metadata=Meta(trajectory_id="a", note="only metadata"))
  w.write_step(**paths(str(tmp_path), "b", 0), metadata=Meta(trajectory_id="b"), step=Step(step_id=0))
  w.write_step(**paths(str(tmp_path), "a", 0), metadata=Meta(trajectory_id="a", note="only metadata"), step=Step(step_id=0))
  w.flush()
  assert order == [("a", None), ("b", "step_0.json"), ("a", "step_0.json")]
  assert os.listdir(tmp_path / "a") and read(tmp_path / "a" / "metadata.json")["note"] == "only metadata"
  w.close()


def test_the_file_holds_what_the_objects_were_at_the_call(tmp_path):
  w = aw.AsyncFileWriter()
  gate = threading.Event()
  real = w._process_task
  w._process_task = lambda task: (gate.wait(2), real(task))[1]
  meta, step = Meta(trajectory_id="t", tags=["x"]), Step(step_id=0, values=[1, 2])
  w.write_step(**paths(str(tmp_path), "t", 0), metadata=meta, step=step)
  step.values.append(3); step.text = "changed"; meta.tags.append("y")        # before the worker got to it
  later = Step(step_id=1, values=step.values)
  w.write_step(**paths(str(tmp_path), "t", 1), metadata=meta, step=later)
  gate.set()
  w.flush()
  assert read(tmp_path / "t" / "step_0.json") == {"step_id": 0, "text": "", "values": [1, 2]}
  assert read(tmp_path / "t" / "step_1.json")["values"] == [1, 2, 3]
  assert read(tmp_path / "t" / "metadata.json")["tags"] == ["x", "y"]
  w.close()


def test_the_thread_starts_on_the_first_write_only_once(tmp_path):
  w = aw.AsyncFileWriter()
  assert w._thread is None
  w.flush(); w.flush()                                            # nothing to wait for, no thread spawned
  assert w._thread is None
  barrier = threading.Barrier(8)

  def racer(k):
    barrier.wait()
    w.write_step(**paths(str(tmp_path), f"t{k}", 0), metadata=Meta(trajectory_id=f"t{k}"), step=Step(step_id=0))
  threads = [threading.Thread(target=racer, args=(k,)) for k in range(8)]
  for t in threads: t.start()
  for t in threads: t.join()
  w.flush()
  assert sum(1 for t in threading.enumerate() if t.name == "trajectory-writer") == 1
  assert sorted(os.listdir(tmp_path)) == [f"t{k}" for k in range(8)]
  w.close()
  untouched = aw.AsyncFileWriter()
  untouched.close(); del untouched                                # closing (or dropping) an unused writer is fine


def test_metadata_is_rewritten_only_when_it_changed(tmp_path):
  w = aw.AsyncFileWriter()
  writes = []
  real = aw.atomic_write_text
  aw.atomic_write_text = lambda path, text: (writes.append(os.path.basename(path)), real(path, text))[1]
  try:
    for k in range(3):
      w.write_step(**paths(str(tmp_path), "t", k), metadata=Meta(trajectory_id="t", note="same"), step=Step(step_id=k))
    w.write_step(**paths(str(tmp_path), "t", 3), metadata=Meta(trajectory_id="t", note="new"), step=Step(step_id=3))
    w.flush()
  finally:
    aw.atomic_write_text = real
  assert writes == ["metadata.json", "step_0.json", "step_1.json", "step_2.json", "metadata.json", "step_3.json"]
  assert read(tmp_path / "t" / "metadata.json")["note"] == "new"
  w.close()


def test_io_errors_are_counted_logged_and_do_not_stop_later_writes(tmp_path, caplog):
  w = aw.AsyncFileWriter()
  blocked = tmp_path / "blocked"
  blocked.write_text("a file where a directory should be")
  with caplog.at_level("ERROR"):
    w.write_step(**paths(str(tmp_path), "blocked", 0), metadata=Meta(trajectory_id="blocked"), step=Step(step_id=0))
    w.write_step(**paths(str(tmp_path), "fine", 0), metadata=Meta(trajectory_id="fine"), step=Step(step_id=0))
    w.flush()
  assert w.errors == 1 and "trajectory write failed" in caplog.text
  assert read(tmp_path / "fine" / "step_0.json")["step_id"] == 0
  w.close()


def test_close_drains_refuses_new_work_and_is_safe_to_repeat_or_race(tmp_path):
  w = aw.AsyncFileWriter()
  real = w._process_task
  w._process_task = lambda task: (time.sleep(0.02), real(task))[1]
  for k in range(5):
    w.write_step(**paths(str(tmp_path), "t", k), metadata=Meta(trajectory_id="t"), step=Step(step_id=k))
  closers = [threading.Thread(target=w.close) for _ in range(4)]
  for t in closers: t.start()
  for t in closers: t.join()
  assert sorted(os.listdir(tmp_path / "t")) == ["metadata.json"] + [f"step_{k}.json" for k in range(5)]   # queued work was written
  with pytest.raises(RuntimeError, match="closed"):
    w.write_step(**paths(str(tmp_path), "t", 9), metadata=Meta(trajectory_id="t"), step=Step(step_id=9))
  w.close(); w.flush()                                            # both return at once


def test_writes_racing_with_close_are_either_written_or_refused_never_lost(tmp_path):
  w = aw.AsyncFileWriter()
  accepted, refused = [], []

  def producer(k):
    for j in range(40):
      try:
        w.write_step(**paths(str(tmp_path), f"p{k}", j), metadata=Meta(trajectory_id=f"p{k}"), step=Step(step_id=j))
        accepted.append((k, j))
      except RuntimeError:
        refused.append((k, j))
  producers = [threading.Thread(target=producer, args=(k,)) for k in range(4)]
  for t in producers: t.start()
  time.sleep(0.005)
  w.close(timeout=10)
  for t in producers: t.join()
  w.flush()                                                       # must not hang on a task queued behind the marker
  assert len(accepted) + len(refused) == 160
  for k, j in accepted:
    assert os.path.exists(tmp_path / f"p{k}" / f"step_{j}.json"), (k, j)


def test_a_stuck_worker_makes_close_warn_instead_of_hanging(tmp_path, caplog):
  w = aw.AsyncFileWriter()
  release = threading.Event()
  w._process_task = lambda task: release.wait(5)
  w.write_step(**paths(str(tmp_path), "t", 0), metadata=Meta(trajectory_id="t"), step=Step(step_id=0))
  with caplog.at_level("WARNING"):
    t0 = time.perf_counter()
    w.close(timeout=0.1)
  assert time.perf_counter() - t0 < 1.0 and "did not finish" in caplog.text
  release.set()
