"""Conformance suite for trajectory stores (tunix/experimental/trajectory/store_testing.py:15-321).

A store implementation proves that it keeps the reader / writer contract by subclassing `StoreConformance` in a
pytest module and providing `make_store`:

    class TestMyStore(store_testing.StoreConformance):
      def make_store(self, tmp_path):
        return MyStore(tmp_path / "root")           # or (reader, writer) when they are two objects

Every test gets a fresh store. What is checked: empty stores, steps coming back in step order whatever the write
order, several trajectories written interleaved, snapshots (the caller may mutate what it handed over), metadata
updates with and without steps, flush being idempotent and harmless on an empty store, ids that are not a single
path component being refused, and the two not-found errors.
"""
from __future__ import annotations

from typing import Any, Tuple

import pytest

from . import store
from . import trajectory as T

BAD_IDS = (None, "", ".", "..", "a/b", "a\\b", "nul\0byte")


def sample_trajectory(trajectory_id: str, turns: int = 2, agent: str = "conformance") -> T.Trajectory:
  traj = T.Trajectory(agent=T.Agent(name=agent, version="1.0"), trajectory_id=trajectory_id)
  for turn in range(turns):
    traj.add_step(T.Source.USER, f"{trajectory_id} question {turn}")
    traj.add_step(T.Source.AGENT, f"{trajectory_id} answer {turn}", model_name="m")
  return traj


def assert_steps_equal(got: T.Step, want: T.Step) -> None:
  assert got.model_dump(exclude={"timestamp"}) == want.model_dump(exclude={"timestamp"})


def assert_trajectories_equal(got: T.Trajectory, want: T.Trajectory) -> None:
  assert got.trajectory_id == want.trajectory_id and got.agent == want.agent
  assert [s.step_id for s in got.steps] == [s.step_id for s in want.steps]
  for a, b in zip(got.steps, want.steps):
    assert_steps_equal(a, b)


class StoreConformance:

  def make_store(self, tmp_path) -> Any:
    raise NotImplementedError

  @pytest.fixture
  def rw(self, tmp_path) -> Tuple[store.TrajectoryReader, store.TrajectoryWriter]:
    made = self.make_store(tmp_path)
    reader, writer = made if isinstance(made, tuple) else (made, made)
    yield reader, writer
    for part in {id(reader): reader, id(writer): writer}.values():
      close = getattr(part, "close", None)
      if callable(close):
        close()

  @staticmethod
  def _write(writer, traj: T.Trajectory, order=None) -> None:
    steps = traj.steps if order is None else [traj.steps[i] for i in order]
    for step in steps:
      writer.add_step(step, traj.get_metadata())

  # ---- reader --------------------------------------------------------------------------------
  def test_protocols(self, rw):
    reader, writer = rw
    assert isinstance(reader, store.TrajectoryReader) and isinstance(writer, store.TrajectoryWriter)

  def test_an_empty_store_lists_nothing_and_finds_nothing(self, rw):
    reader, writer = rw
    writer.flush()                                     # nothing pending: harmless
    assert reader.get_trajectories_metadata() == [] and reader.get_trajectories([]) == []
    with pytest.raises(store.TrajectoryNotFoundError) as e:
      reader.get_trajectories(["missing"])
    assert e.value.trajectory_id == "missing" and isinstance(e.value, KeyError)

  def test_steps_come_back_in_step_order_whatever_the_write_order(self, rw):
    reader, writer = rw
    traj = sample_trajectory("t1", turns=2)
    self._write(writer, traj, order=[2, 0, 3, 1])
    writer.flush()
    (got,) = reader.get_trajectories(["t1"])
    assert_trajectories_equal(got, traj)

  def test_trajectories_written_interleaved_stay_apart_and_load_in_the_order_asked(self, rw):
    reader, writer = rw
    a, b = sample_trajectory("a", turns=1), sample_trajectory("b", turns=3)
    for i in range(6):
      if i < len(a.steps):
        writer.add_step(a.steps[i], a.get_metadata())
      writer.add_step(b.steps[i], b.get_metadata())
    writer.flush()
    assert sorted(m.trajectory_id for m in reader.get_trajectories_metadata()) == ["a", "b"]
    got_b, got_a = reader.get_trajectories(["b", "a"])
    assert_trajectories_equal(got_a, a)
    assert_trajectories_equal(got_b, b)
    with pytest.raises(store.TrajectoryNotFoundError):
      reader.get_trajectories(["a", "c"])

  # ---- writer --------------------------------------------------------------------------------
  def test_the_store_keeps_a_snapshot_of_what_it_was_given(self, rw):
    reader, writer = rw
    traj = sample_trajectory("snap", turns=1)
    meta = traj.get_metadata()
    meta.notes = "as written"
    for step in traj.steps:
      writer.add_step(step, meta)
      step.message = "changed after the call"
    meta.notes = "changed after the call"
    writer.flush()
    (got,) = reader.get_trajectories(["snap"])
    assert [s.message for s in got.steps] == ["snap question 0", "snap answer 0"] and got.notes == "as written"

  def test_a_later_metadata_wins_and_needs_no_steps(self, rw):
    reader, writer = rw
    traj = sample_trajectory("m", turns=1)
    self._write(writer, traj)
    meta = traj.get_metadata()
    meta.notes = "final"
    meta.final_metrics = T.FinalMetrics(total_steps=2)
    writer.update_metadata(meta)
    meta.notes = "changed after the call"
    bare = T.TrajectoryMetadata(agent=T.Agent(name="conformance"), trajectory_id="bare")
    writer.update_metadata(bare)
    writer.flush()
    by_id = {m.trajectory_id: m for m in reader.get_trajectories_metadata()}
    assert by_id["m"].notes == "final" and by_id["m"].final_metrics.total_steps == 2 and "bare" in by_id
    (got,) = reader.get_trajectories(["bare"])
    assert got.steps == [] and got.agent.name == "conformance"

  def test_rewriting_a_step_replaces_it_and_flush_is_idempotent(self, rw):
    reader, writer = rw
    traj = sample_trajectory("r", turns=1)
    self._write(writer, traj)
    writer.flush()
    again = traj.steps[1].model_copy(update={"message": "second thoughts"})
    writer.add_step(again, traj.get_metadata())
    writer.flush()
    writer.flush()
    (got,) = reader.get_trajectories(["r"])
    assert [s.message for s in got.steps] == ["r question 0", "second thoughts"]

  @pytest.mark.parametrize("bad", BAD_IDS)
  def test_ids_that_are_not_one_path_component_are_refused(self, rw, bad):
    reader, writer = rw
    meta = T.TrajectoryMetadata(agent=T.Agent(name="x"), trajectory_id=bad)
    with pytest.raises(ValueError):
      writer.add_step(T.Step(step_id=1, source=T.Source.USER, message="m"), meta)
    with pytest.raises(ValueError):
      writer.update_metadata(meta)
    writer.flush()
    assert reader.get_trajectories_metadata() == []
