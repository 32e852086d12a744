"""Remote execution beyond the happy path: wire objects, server-side error reporting, background tasks and polling,
routing policies, dynamic sessions with fault isolation, the decorator's argument checks, and gRPC with large payloads."""
import asyncio
import threading
import time

import numpy as np
import pytest

from tunix_b200.experimental.worker import remote_execution as rx


class Worker:
  def __init__(self, name="w", delay=0.0):
    self.name, self.delay, self.calls = name, delay, 0

  def who(self, *args, **kwargs):
    self.calls += 1
    return self.name

  def echo(self, x):
    return x

  async def slow(self, x):
    await asyncio.sleep(self.delay or 0.01)
    return (self.name, x)

  def boom(self, what="bad"):
    raise LookupError(what)

  def lock(self):
    return threading.Lock()

  def __call__(self, x):
    return ("called", x)


def handle(*a, **k):
  return rx.InProcessActorHandle(rx.InProcessRemoteExecutionServer(Worker(*a, **k)))


# ---- wire objects -----------------------------------------------------------------------------------
def test_request_and_response_round_trip_and_defaults():
  req = rx.ExecutionRequest("id-1", "echo", [1, "two"], {"k": np.arange(3)})
  back = rx.ExecutionRequest.deserialize(req.serialize())
  assert (back.request_id, back.method_name, back.args[:2]) == ("id-1", "echo", (1, "two"))
  assert back.kwargs["k"].tolist() == [0, 1, 2]
  bare = rx.ExecutionRequest()
  assert bare.method_name == "__call__" and bare.args == () and bare.kwargs == {} and bare.request_id is None
  ok = rx.ExecutionResponse.deserialize(rx.ExecutionResponse(result={"a": 1}, request_id="r").serialize())
  assert ok.unwrap() == {"a": 1} and ok.request_id == "r" and ok.error_message is None
  try:
    raise KeyError("missing")
  except KeyError as e:
    failed = rx.ExecutionResponse.from_exception(e, "r2")
  failed = rx.ExecutionResponse.deserialize(failed.serialize())
  assert failed.error_type == "KeyError" and "test_remote_execution.py" in failed.traceback and not failed.retryable
  with pytest.raises(RuntimeError, match=r"(?s)RemoteExecutionError \[KeyError\].*Remote traceback"):
    failed.unwrap()


def test_default_method_is_the_call_operator():
  assert handle().submit(None, 5) == ("called", 5)
  assert asyncio.run(handle().asubmit(None, 6)) == ("called", 6)


# ---- what the server reports ----------------------------------------------------------------------
def test_server_errors_are_responses_not_exceptions():
  empty = rx.InProcessRemoteExecutionServer()
  req = rx.ExecutionRequest("x", "who")
  for response in (empty.execute_sync_request(req), asyncio.run(empty.execute_request(req))):
    assert response.error_type == "InstanceNotBoundError" and response.request_id == "x"
  empty.register_instance(Worker())
  assert empty.bound_instance.name == "w" and empty.execute_sync_request(req).unwrap() == "w"
  for response in (empty.execute_sync_request(rx.ExecutionRequest("y", "nope")),
                   asyncio.run(empty.execute_request(rx.ExecutionRequest("y", "name")))):      # an attribute, not a method
    assert response.error_type == "AttributeError" and "not found" in response.error_message
  sync_on_coroutine = empty.execute_sync_request(rx.ExecutionRequest("z", "slow", [1]))
  assert "coroutine function" in sync_on_coroutine.error_message
  raised = empty.execute_sync_request(rx.ExecutionRequest("e", "boom", kwargs={"what": "kaput"}))
  assert raised.error_type == "LookupError" and raised.error_message == "kaput" and "boom" in raised.traceback
  unpicklable = rx.ExecutionResponse.deserialize(empty.execute_sync_request(rx.ExecutionRequest("l", "lock")).serialize())
  assert unpicklable.error_type == "ExecutionResponseSerializationError" and unpicklable.result is None


def test_coroutine_methods_through_the_synchronous_entry():
  h = handle()
  assert h.submit("slow", 3) == ("w", 3)                 # no loop running: the handle runs one

  async def inside():
    with pytest.raises(RuntimeError, match="use asubmit"):
      h.submit("slow", 3)
    return await h.asubmit("slow", 4)
  assert asyncio.run(inside()) == ("w", 4)


def test_background_tasks_ids_polling_and_timeouts():
  async def scenario():
    h = handle(delay=0.02)
    assert await h.poll_responses(timeout_s=0.0) == [] and await h.poll_responses(timeout_s=0.02) == []
    auto = [await h.dispatch_task(None, "slow", i) for i in range(2)]
    custom = await h.dispatch_task("mine", "boom")
    assert auto == ["task_1", "task_2"] and custom == "mine"
    got = []
    deadline = time.monotonic() + 2
    while len(got) < 3 and time.monotonic() < deadline:
      got += await h.poll_responses(timeout_s=0.2, max_items=2)
    by_id = {r.request_id: r for r in got}
    assert sorted(by_id) == ["mine", "task_1", "task_2"]
    assert by_id["task_2"].unwrap() == ("w", 1) and by_id["mine"].error_type == "LookupError"
    assert await h.poll_responses(timeout_s=0.0) == []
    # a task whose result is None is still a response
    await h.dispatch_task("none", "echo", None)
    (only,) = await h.poll_responses(timeout_s=1.0)
    assert only.request_id == "none" and only.unwrap() is None
  asyncio.run(scenario())


# ---- routing ----------------------------------------------------------------------------------------
def test_pool_argument_checks():
  pool = rx.RoutingActorPool()
  with pytest.raises(RuntimeError, match="no registered ActorHandles"):
    pool.submit("who")

  async def stream():
    async for _ in pool.as_completed_stream([("a", "who", (), {})]):
      pass
  with pytest.raises(RuntimeError, match="no registered ActorHandles"):
    asyncio.run(stream())
  with pytest.raises(TypeError, match="Expected str or ActorHandle"):
    pool.add_actor(42)
  with pytest.raises(ValueError, match="unknown routing policy"):
    rx.RoutingActorPool(policy="random")
  pool.add_actor(handle("solo"))
  assert pool.submit("who") == "solo" and len(pool.actors) == 1


def test_routing_keys_are_stable_and_removed_before_the_call():
  hs = [handle(f"w{i}") for i in range(4)]
  pool = rx.RoutingActorPool(hs)
  first = [pool.submit("who", route_key=f"user-{i}") for i in range(20)]
  again = [pool.submit("who", route_key=f"user-{i}") for i in range(20)]
  assert first == again and len(set(first)) > 1          # sticky per key, spread over actors
  # the choice is a CRC of the key, so it is the same in another process or run
  import zlib
  assert first[3] == f"w{zlib.crc32(repr('user-3').encode()) % 4}"


def test_least_loaded_prefers_idle_actors_and_routers_can_be_objects():
  slow, fast = handle("slow", delay=0.2), handle("fast", delay=0.0)
  pool = rx.RoutingActorPool([slow, fast], policy="least_loaded")

  async def scenario():
    busy = asyncio.create_task(pool.asubmit("slow", 0))       # occupies the first actor
    await asyncio.sleep(0.02)
    picks = [await pool.asubmit("who") for _ in range(3)]
    await busy
    return picks
  assert asyncio.run(scenario()) == ["fast", "fast", "fast"]

  class ByMethod:
    def who(self, actors, args, kwargs):
      return actors[1]
  routed = rx.RoutingActorPool([slow, fast], router=ByMethod())
  assert routed.submit("who") == "fast"
  with pytest.raises(TypeError, match="must provide a method matching 'echo' or be callable"):
    routed.submit("echo", 1)


# ---- sessions ---------------------------------------------------------------------------------------
def test_session_accepts_new_work_while_draining_and_isolates_failures():
  pool = rx.RoutingActorPool([handle("a", delay=0.01), handle("b", delay=0.01)])

  async def scenario():
    results, errors, spawned = [], [], 0
    async with pool.execution_session([("first", "slow", (0,), {})]) as session:
      await session.submit("fail", "boom")
      async for value, exc in session.as_completed():
        if exc is not None:
          errors.append(str(exc))
          continue
        results.append(value[1])
        if spawned < 3:                                         # every finished task enqueues a follow-up
          spawned += 1
          await session.submit(None, "slow", value[1] + 1)
      with pytest.raises(RuntimeError, match="closed"):
        await session.close() or await session.submit(None, "who")
    return results, errors
  results, errors = asyncio.run(scenario())
  assert sorted(results) == [0, 1, 2, 3] and len(errors) == 1 and "LookupError" in errors[0]
  assert all(v == 0 for v in pool._inflight.values())           # load counters are back to zero


def test_a_dispatch_that_fails_is_not_counted_as_in_flight():
  class Broken(rx.InProcessActorHandle):
    async def dispatch_task(self, *a, **k):
      raise ConnectionError("actor unreachable")
  pool = rx.RoutingActorPool([Broken(rx.InProcessRemoteExecutionServer(Worker())), handle("ok")])

  async def scenario():
    async with pool.execution_session() as session:
      with pytest.raises(ConnectionError):
        await session.submit("t0", "who")                       # round robin: the broken actor first
      await session.submit("t1", "who")
      return [item async for item in session.as_completed()]
  assert asyncio.run(scenario()) == [("ok", None)]
  assert all(v == 0 for v in pool._inflight.values())


def test_one_shot_stream_raises_the_first_failure():
  pool = rx.RoutingActorPool([handle("a")])

  async def scenario(tasks):
    return [r async for r in pool.as_completed_stream(tasks)]
  assert asyncio.run(scenario([])) == []
  assert asyncio.run(scenario([("x", "echo", (None,), {}), ("y", "echo", (2,), {})])) in ([None, 2], [2, None])
  with pytest.raises(RuntimeError, match="LookupError"):
    asyncio.run(scenario([("x", "boom", (), {})]))


# ---- decorator ----------------------------------------------------------------------------------------
def test_remote_decorator_forms_and_argument_checks():
  @rx.remote
  class Counter:
    """doc kept"""
    def __init__(self, start): self.n = start
    def inc(self): self.n += 1; return self.n
  h = Counter.remote(5)
  assert isinstance(h, rx.ActorHandle) and h.submit("inc") == 6 and Counter.__doc__ == "doc kept"
  assert Counter.__name__ == "Counter" and Counter.__wrapped__(1).inc() == 2

  @rx.remote
  async def twice(x):
    return 2 * x
  assert twice.remote(4) == 8 and asyncio.run(_await(twice.remote, 5)) == 10

  @rx.remote(transport="carrier-pigeon")
  class Odd:
    pass
  with pytest.raises(ValueError, match="Unsupported transport"):
    Odd.remote()
  with pytest.raises(NotImplementedError, match="standalone functions"):
    rx.remote(transport="grpc")(lambda: 1)
  with pytest.raises(TypeError, match="expects a class or function"):
    rx.remote(42)
  by_address = rx.remote("grpc://127.0.0.1:1")(Worker)
  assert isinstance(by_address.remote(), rx.GrpcRemoteActorHandle)


async def _await(fn, *a):
  return await fn(*a)


# ---- gRPC -----------------------------------------------------------------------------------------------
def test_grpc_large_payloads_repeated_calls_and_remote_tracebacks():
  pytest.importorskip("grpc")
  server = rx.GrpcRemoteExecutionServer(Worker("remote"))
  server.start_serving(port=0)
  h = rx.ActorHandle.from_address(f"grpc://127.0.0.1:{server.port}")
  try:
    big = np.random.default_rng(0).integers(0, 255, 8 << 20, dtype=np.uint8)        # 8 MiB each way
    back = h.submit("echo", big)
    assert back.shape == big.shape and np.array_equal(back, big)
    assert [h.submit("who") for _ in range(20)] == ["remote"] * 20
    with pytest.raises(RuntimeError, match=r"RemoteExecutionError \[LookupError\]: far away"):
      h.submit("boom", what="far away")
    with pytest.raises(RuntimeError, match="ExecutionResponseSerializationError"):
      h.submit("lock")
    assert h.submit("who") == "remote"                                             # the channel survived all of it
  finally:
    asyncio.run(h.close())
    server.shutdown()
