"""More scenarios of the weight-sync coordinator: ordering and concurrency of phases, identity of rounds, publish
retries, uniform rollback, serialisation of rounds, and what a cancelled round leaves behind."""
import asyncio
import time

import pytest
import torch

from tunix_b200.experimental.orchestrator import peer_memory_handler, weight_sync, weight_sync_coordinator as wsc
from tests.test_control_plane import FakeDest, FakeSource, make_round


def run(coro):
  return asyncio.run(coro)


def test_phases_arrive_in_order_and_destinations_work_concurrently():
  h, src, dests, co = make_round()
  log = []
  for d in dests:
    original = d._phase

    async def slow(name, phase, req, work, d=d, original=original):
      log.append((name, d.wid, "start"))
      await asyncio.sleep(0.05)
      await original(name, phase, req, work)
      log.append((name, d.wid, "end"))
    d._phase = slow
  t0 = time.perf_counter()
  assert run(co.sync(1)).success
  took = time.perf_counter() - t0
  assert took < 3 * 0.05 * 2 * 0.9                      # three phases, two workers each: overlapped, not serial
  order = [n for n, _, edge in log if edge == "start"]
  assert order == ["pre_weight_sync"] * 2 + ["weight_sync"] * 2 + ["post_weight_sync"] * 2
  # within a phase both workers had started before either finished
  for phase in ("pre_weight_sync", "weight_sync", "post_weight_sync"):
    edges = [edge for n, _, edge in log if n == phase]
    assert edges == ["start", "start", "end", "end"]


def test_every_round_has_its_own_identity_even_for_a_retried_version():
  h, src, dests, co = make_round(fail=[set(), {"pre_weight_sync"}])
  first = run(co.sync(1, raise_on_failure=False))
  dests[1].fail = set()
  second = run(co.sync(1, raise_on_failure=False))              # the same version again: allowed after an abort
  assert first.state == wsc.RoundState.ABORTED and second.success
  assert (first.req_id, first.uuid) != (second.req_id, second.uuid) and second.uuid == first.uuid + 1
  assert second.round_index == 2 and co.last_result is second
  assert [u.job_name for u in second.source_units] == ["trainer"] and len(second.destination_units) == 2
  assert second.transfer.success and "bytes" in second.transfer.message


def test_source_is_prepared_once_and_released_on_every_path():
  h, src, dests, co = make_round()
  calls = []
  real = src.prepare_weight_sync

  async def counting(req=None, **kw):
    calls.append(req.extra_config["uuid"])
    return await real(req, **kw)
  src.prepare_weight_sync = counting
  run(co.sync(1))
  assert calls == [1] and src.released == 1
  dests[0].fail = {"weight_sync"}
  run(co.sync(2, raise_on_failure=False))
  assert calls == [1, 2] and src.released == 2                  # the failure path released it too


def test_transient_publish_failure_is_retried_to_commit():
  h, src, dests, co = make_round()
  flaky = dests[1]
  real = flaky.post_weight_sync
  attempts = []

  async def once_broken(req=None):
    attempts.append(1)
    if len(attempts) == 1:
      raise TimeoutError("publish RPC timed out before it reached the worker")
    await real(req)
  flaky.post_weight_sync = once_broken
  res = run(co.sync(1))
  assert res.success and len(attempts) == 2 and all(d.version == 1 for d in dests) and not co.poisoned
  # without retries the same fault splits the fleet
  h, src, dests, co2 = make_round()
  co2 = wsc.WeightSyncCoordinator(h, sources=[src], destinations=dests, post_retries=0)
  attempts.clear()
  real2 = dests[1].post_weight_sync

  async def once_broken2(req=None):
    attempts.append(1)
    if len(attempts) == 1:
      raise TimeoutError("lost")
    await real2(req)
  dests[1].post_weight_sync = once_broken2
  assert run(co2.sync(1, raise_on_failure=False)).state == wsc.RoundState.PARTIALLY_COMMITTED


def test_publish_failing_everywhere_rolls_back_uniformly_and_does_not_poison():
  h, src, dests, co = make_round(fail={"post_weight_sync"})
  res = run(co.sync(1, raise_on_failure=False))
  assert res.state == wsc.RoundState.ABORTED and co.poisoned is None
  assert all(d.version == 0 and d.admitting and d.serving["w"][0, 0] == -1.0 for d in dests)
  assert {r.phase for r in res.workers} == {"aborted"} and src.released == 1
  for d in dests:
    d.fail = set()
  assert run(co.sync(1)).success                                # the coordinator is still usable


def test_rounds_do_not_interleave():
  h, src, dests, co = make_round()
  active, overlaps = [], []
  real = dests[0].pre_weight_sync

  async def watching(req=None):
    active.append(req.extra_config["uuid"])
    overlaps.append(len(active))
    await asyncio.sleep(0.05)
    await real(req)
    active.remove(req.extra_config["uuid"])
  dests[0].pre_weight_sync = watching

  async def two():
    return await asyncio.gather(co.sync(1), co.sync(2))
  a, b = run(two())
  assert a.success and b.success and overlaps == [1, 1] and co.last_committed_version == 2
  assert sorted([a.uuid, b.uuid]) == [1, 2]


def test_a_destination_without_the_protocol_fails_before_any_downtime():
  h, src, dests, co = make_round()

  class NotADestination:
    def info(self):
      return dests[0].info()
  co = wsc.WeightSyncCoordinator(h, sources=[src], destinations=[dests[0], NotADestination()])
  res = run(co.sync(1, raise_on_failure=False))
  assert res.state == wsc.RoundState.ABORTED and "preparation failed" in res.failures[0]
  assert dests[0].calls == [] and dests[0].admitting
  with pytest.raises(ValueError, match="no weight-sync destination"):
    run(wsc.WeightSyncCoordinator(h, sources=[src], destinations=[]).sync(1))


# ---- cancellation ----------------------------------------------------------------------------------
def _cancel_when(co, dests, src, phase_name, where="dest"):
  """Runs a round and cancels its task once `phase_name` has started on the first destination (or, for
  "transfer", inside the handler)."""
  async def scenario():
    started = asyncio.Event()
    loop = asyncio.get_running_loop()
    if phase_name == "transfer":
      real_transfer = co._handler.transfer

      def slow_transfer(*a, **k):
        loop.call_soon_threadsafe(started.set)
        time.sleep(0.2)
        return real_transfer(*a, **k)
      co._handler.transfer = slow_transfer
    else:
      real = getattr(dests[0], phase_name)

      async def slow(req=None):
        started.set()
        await asyncio.sleep(0.2)
        await real(req)
      setattr(dests[0], phase_name, slow)
    task = asyncio.create_task(co.sync(1))
    await started.wait()
    task.cancel()
    with pytest.raises(asyncio.CancelledError):
      await task
    await asyncio.sleep(0.3)                    # lets a transfer thread that is still running finish
  run(scenario())


@pytest.mark.parametrize("phase", ["pre_weight_sync", "weight_sync"])
def test_cancelled_before_the_publish_rolls_everything_back(phase):
  h, src, dests, co = make_round()
  _cancel_when(co, dests, src, phase)
  res = co.last_result
  assert res.state == wsc.RoundState.ABORTED and f"cancelled during" in res.failures[0]
  assert all(d.admitting and d.version == 0 for d in dests) and src.released == 1 and co.poisoned is None
  assert all("abort_weight_sync" in d.calls for d in dests)
  assert run(co.sync(1)).success                                # and the next round works


def test_cancelled_during_the_transfer_parks_the_round_and_touches_nothing():
  h, src, dests, co = make_round()
  _cancel_when(co, dests, src, "transfer")
  res = co.last_result
  assert res.state == wsc.RoundState.UNKNOWN_TRANSFER_STATE and co.poisoned
  assert src.released == 0 and all("abort_weight_sync" not in d.calls and not d.admitting for d in dests)
  assert all(r.needs_restart for r in res.workers)
  with pytest.raises(RuntimeError, match="poisoned"):
    run(co.sync(2))


def test_cancelled_during_the_publish_still_converges_on_the_new_version():
  h, src, dests, co = make_round()
  src.weights["w"].fill_(7.0)
  _cancel_when(co, dests, src, "post_weight_sync")
  res = co.last_result
  assert res.state == wsc.RoundState.COMMITTED and co.last_committed_version == 1 and not co.poisoned
  assert all(d.version == 1 and d.admitting and d.serving["w"][0, 0] == 7.0 for d in dests)
  assert src.released == 1 and "cancelled during publish" in res.failures[0]


def test_cancelled_publish_with_a_broken_worker_is_reported_partial():
  h, src, dests, co = make_round(fail=[set(), {"post_weight_sync"}])
  _cancel_when(co, dests, src, "post_weight_sync")
  res = co.last_result
  assert res.state == wsc.RoundState.PARTIALLY_COMMITTED and co.poisoned
  assert dests[0].version == 1 and dests[1].version == 0
  assert [r.worker_id for r in res.workers if r.needs_restart] == ["r1"]
