"""Method calls on objects that live in another process (tunix/experimental/worker/remote_execution.py:104-1280).

A `RemoteExecutionServer` binds one object and executes `(method name, args, kwargs)` envelopes
against it; an `ActorHandle` is the caller's side: `submit` (blocking), `asubmit` (awaitable),
and the fire-and-collect pair `dispatch_task` / `poll_responses` for long calls. Envelopes are
cloudpickle bytes. Transports: in-process (same interpreter, used by tests and single-process
runs) and gRPC with byte payloads over generic method handlers, so no generated stubs are
needed. A remote failure comes back as a structured error and is re-raised by `unwrap()` with
the remote traceback attached. `RoutingActorPool` spreads calls over handles (custom router,
sticky `route_key`, least-loaded or round-robin); `PoolExecutionSession` streams results of
many dispatched tasks as they finish, isolating per-task failures; `@remote` turns a class
or function into a factory of handles.
"""
from __future__ import annotations

import abc
import asyncio
import contextlib
import inspect
import zlib
import threading
import traceback as traceback_lib
from typing import Any, AsyncIterator, Callable, Dict, List, Optional, Sequence, Tuple, Union

import cloudpickle

LONG_POLL_TIMEOUT_S = 30.0
_SERVICE = "tunix_b200.RemoteExecution"
_MAX_MSG = 1 << 30


class ExecutionRequest:
  def __init__(self, request_id: Optional[str] = None, method_name: Optional[str] = None,
               args: Optional[Sequence[Any]] = None, kwargs: Optional[Dict[str, Any]] = None):
    self.request_id = request_id
    self.method_name = method_name or "__call__"
    self.args: Tuple[Any, ...] = tuple(args or ())
    self.kwargs: Dict[str, Any] = dict(kwargs or {})
    if "request_id" in self.kwargs:
      raise ValueError("'request_id' is a reserved framework parameter for remote execution and cannot be passed in "
                       "method kwargs.")

  def serialize(self) -> bytes:
    return cloudpickle.dumps((self.request_id, self.method_name, self.args, self.kwargs))

  @classmethod
  def deserialize(cls, payload: bytes) -> "ExecutionRequest":
    rid, name, args, kwargs = cloudpickle.loads(payload)
    return cls(rid, name, args, kwargs)


class ExecutionResponse:
  def __init__(self, result: Any = None, error_message: Optional[str] = None, error_type: Optional[str] = None,
               traceback: Optional[str] = None, retryable: bool = False, request_id: Optional[str] = None):
    self.result, self.error_message, self.error_type = result, error_message, error_type
    self.traceback, self.retryable, self.request_id = traceback, retryable, request_id

  def _tuple(self):
    return (self.result, self.error_message, self.error_type, self.traceback, self.retryable, self.request_id)

  def serialize(self) -> bytes:
    try:
      return cloudpickle.dumps(self._tuple())
    except Exception as e:          # an unpicklable result must not take the channel down
      self.error_message = f"failed to serialize result of type {type(self.result).__name__}: {e}"
      self.result, self.error_type = None, "ExecutionResponseSerializationError"
      self.traceback, self.retryable = traceback_lib.format_exc(), False
      return cloudpickle.dumps(self._tuple())

  @classmethod
  def deserialize(cls, payload: bytes) -> "ExecutionResponse":
    return cls(*cloudpickle.loads(payload))

  @classmethod
  def from_exception(cls, e: BaseException, request_id: Optional[str]) -> "ExecutionResponse":
    return cls(error_message=str(e), error_type=type(e).__name__, traceback=traceback_lib.format_exc(),
               request_id=request_id)

  def unwrap(self) -> Any:
    if self.error_message is not None:
      msg = f"RemoteExecutionError [{self.error_type}]: {self.error_message}"
      if self.traceback:
        msg += f"\nRemote traceback:\n{self.traceback}"
      raise RuntimeError(msg)
    return self.result


# ---- server -------------------------------------------------------------------------------------
class RemoteExecutionServer(abc.ABC):
  def __init__(self, instance: Optional[Any] = None):
    self._instance = instance
    self._responses: Optional[asyncio.Queue] = None
    self._responses_loop: Optional[asyncio.AbstractEventLoop] = None
    self._counter = 0
    self._background: set = set()

  def register_instance(self, instance: Any) -> None:
    self._instance = instance

  @property
  def bound_instance(self) -> Optional[Any]:
    return self._instance

  @abc.abstractmethod
  def start_serving(self, port: int) -> None: ...

  def _queue(self) -> asyncio.Queue:
    """The response queue of the running loop. An asyncio queue belongs to the loop that first waited on it; a
    server that outlives a loop (a second `asyncio.run`, a restarted serving thread) gets a fresh queue, and
    responses nobody collected move over."""
    loop = asyncio.get_running_loop()
    if self._responses is None or self._responses_loop is not loop:
      fresh: asyncio.Queue = asyncio.Queue()
      while self._responses is not None and not self._responses.empty():
        fresh.put_nowait(self._responses.get_nowait())
      self._responses, self._responses_loop = fresh, loop
    return self._responses

  def _resolve(self, request: ExecutionRequest):
    """-> (callable, None) or (None, error response)."""
    if self._instance is None:
      return None, ExecutionResponse(error_message="RemoteExecutionServer has no registered instance.",
                                     error_type="InstanceNotBoundError", request_id=request.request_id)
    fn = getattr(self._instance, request.method_name, None)
    if fn is None or not callable(fn):
      return None, ExecutionResponse(error_message=f"Method '{request.method_name}' not found on bound instance.",
                                     error_type="AttributeError", request_id=request.request_id)
    return fn, None

  def execute_sync_request(self, request: ExecutionRequest) -> ExecutionResponse:
    fn, err = self._resolve(request)
    if err is not None:
      return err
    if inspect.iscoroutinefunction(fn):
      return ExecutionResponse(error_message=f"Method '{request.method_name}' is a coroutine function; use asubmit().",
                               error_type="RuntimeError", request_id=request.request_id)
    try:
      return ExecutionResponse(result=fn(*request.args, **request.kwargs), request_id=request.request_id)
    except Exception as e:
      return ExecutionResponse.from_exception(e, request.request_id)

  async def execute_request(self, request: ExecutionRequest) -> ExecutionResponse:
    """Coroutine methods are awaited; plain methods run on the loop's executor so a long call
    does not stall other requests."""
    fn, err = self._resolve(request)
    if err is not None:
      return err
    try:
      if inspect.iscoroutinefunction(fn):
        result = await fn(*request.args, **request.kwargs)
      else:
        result = await asyncio.get_running_loop().run_in_executor(None, lambda: fn(*request.args, **request.kwargs))
        if inspect.isawaitable(result):
          result = await result
      return ExecutionResponse(result=result, request_id=request.request_id)
    except Exception as e:
      return ExecutionResponse.from_exception(e, request.request_id)

  async def dispatch_task(self, request: ExecutionRequest) -> str:
    """Starts the call in the background; its response is collected with `poll_response`."""
    if not request.request_id:
      self._counter += 1
      request.request_id = f"task_{self._counter}"

    async def run():
      await self._queue().put(await self.execute_request(request))
    t = asyncio.create_task(run())
    self._background.add(t)
    t.add_done_callback(self._background.discard)
    return request.request_id

  async def poll_response(self, timeout_s: float = LONG_POLL_TIMEOUT_S) -> Optional[ExecutionResponse]:
    try:
      if timeout_s == 0.0:
        return self._queue().get_nowait()
      return await asyncio.wait_for(self._queue().get(), timeout=timeout_s)
    except (asyncio.TimeoutError, asyncio.QueueEmpty):
      return None


class InProcessRemoteExecutionServer(RemoteExecutionServer):
  def start_serving(self, port: int = 0) -> None:
    return None


class GrpcRemoteExecutionServer(RemoteExecutionServer):
  """Serves `Execute`, `DispatchTask` (unary) and `PollResponses` (server streaming)."""

  def __init__(self, instance: Optional[Any] = None):
    super().__init__(instance)
    self._server = None
    self._loop: Optional[asyncio.AbstractEventLoop] = None
    self._thread: Optional[threading.Thread] = None
    self.port: Optional[int] = None

  async def _execute(self, payload: bytes, context) -> bytes:
    return (await self.execute_request(ExecutionRequest.deserialize(payload))).serialize()

  async def _dispatch(self, payload: bytes, context) -> bytes:
    return cloudpickle.dumps(await self.dispatch_task(ExecutionRequest.deserialize(payload)))

  async def _poll(self, payload: bytes, context):
    timeout_s, max_items = cloudpickle.loads(payload)
    first = await self.poll_response(timeout_s)
    n = 0
    while first is not None and n < max_items:
      yield first.serialize()
      n += 1
      first = await self.poll_response(0.0)

  async def start_serving_async(self, port: int = 50051, host: str = "127.0.0.1"):
    import grpc
    ident = lambda b: b
    handlers = {
        "Execute": grpc.unary_unary_rpc_method_handler(self._execute, ident, ident),
        "DispatchTask": grpc.unary_unary_rpc_method_handler(self._dispatch, ident, ident),
        "PollResponses": grpc.unary_stream_rpc_method_handler(self._poll, ident, ident),
    }
    self._server = grpc.aio.server(options=[("grpc.max_send_message_length", _MAX_MSG),
                                            ("grpc.max_receive_message_length", _MAX_MSG)])
    self._server.add_generic_rpc_handlers((grpc.method_handlers_generic_handler(_SERVICE, handlers),))
    self.port = self._server.add_insecure_port(f"{host}:{port}")
    await self._server.start()
    self._loop = asyncio.get_running_loop()
    return self._server

  def start_serving(self, port: int = 50051, host: str = "127.0.0.1") -> None:
    """Serves from a background thread with its own event loop; returns once listening."""
    ready = threading.Event()
    err: List[BaseException] = []

    def run():
      loop = asyncio.new_event_loop()
      asyncio.set_event_loop(loop)
      try:
        loop.run_until_complete(self.start_serving_async(port, host))
      except BaseException as e:
        err.append(e)
        ready.set()
        return
      ready.set()
      loop.run_forever()
    self._thread = threading.Thread(target=run, daemon=True, name="remote-execution-server")
    self._thread.start()
    ready.wait()
    if err:
      raise err[0]

  @property
  def serve_loop(self) -> Optional[asyncio.AbstractEventLoop]:
    return self._loop

  async def stop_serving(self, grace: float = 0.5) -> None:
    if self._server is not None:
      await self._server.stop(grace)
      self._server = None

  def shutdown(self, grace: float = 0.5) -> None:
    if self._loop is not None and self._server is not None:
      asyncio.run_coroutine_threadsafe(self.stop_serving(grace), self._loop).result(timeout=grace + 5)
      self._loop.call_soon_threadsafe(self._loop.stop)


# ---- handles ------------------------------------------------------------------------------------
class ActorHandle(abc.ABC):
  @staticmethod
  def from_address(address: str) -> "ActorHandle":
    scheme, _, rest = address.partition("://")
    if not rest:
      scheme, rest = "grpc", address
    if scheme == "grpc":
      return GrpcRemoteActorHandle(rest)
    raise ValueError(f"Unsupported actor address scheme {scheme!r} in {address!r}")

  @abc.abstractmethod
  def submit(self, method_name: Optional[str] = None, *args, **kwargs) -> Any: ...

  @abc.abstractmethod
  async def asubmit(self, method_name: Optional[str] = None, *args, **kwargs) -> Any: ...

  @abc.abstractmethod
  async def dispatch_task(self, request_id: Optional[str], method_name: str, *args, **kwargs) -> str: ...

  @abc.abstractmethod
  async def poll_responses(self, timeout_s: float = LONG_POLL_TIMEOUT_S, max_items: int = 64
                           ) -> List[ExecutionResponse]: ...

  async def close(self) -> None:
    return None


class InProcessActorHandle(ActorHandle):
  def __init__(self, server: RemoteExecutionServer):
    self.server = server

  def submit(self, method_name: Optional[str] = None, *args, **kwargs) -> Any:
    req = ExecutionRequest(method_name=method_name, args=args, kwargs=kwargs)
    fn, err = self.server._resolve(req)
    if err is None and inspect.iscoroutinefunction(fn):
      try:
        asyncio.get_running_loop()
      except RuntimeError:
        return asyncio.run(self.server.execute_request(req)).unwrap()
      raise RuntimeError(f"Method '{req.method_name}' is a coroutine function; use asubmit() inside an event loop.")
    return self.server.execute_sync_request(req).unwrap()

  async def asubmit(self, method_name: Optional[str] = None, *args, **kwargs) -> Any:
    return (await self.server.execute_request(ExecutionRequest(method_name=method_name, args=args,
                                                               kwargs=kwargs))).unwrap()

  async def dispatch_task(self, request_id, method_name, *args, **kwargs) -> str:
    return await self.server.dispatch_task(ExecutionRequest(request_id, method_name, args, kwargs))

  async def poll_responses(self, timeout_s: float = LONG_POLL_TIMEOUT_S, max_items: int = 64):
    out = []
    r = await self.server.poll_response(timeout_s)
    while r is not None and len(out) < max_items:
      out.append(r)
      r = await self.server.poll_response(0.0) if len(out) < max_items else None
    return out


class GrpcRemoteActorHandle(ActorHandle):
  """Client of `GrpcRemoteExecutionServer`. Blocking `submit` uses a sync channel; the async
  methods use an aio channel bound to the loop that first uses them."""

  def __init__(self, target: str):
    self.target = target
    self._sync_channel = None
    self._aio: Dict[int, Any] = {}

  @staticmethod
  def _opts():
    return [("grpc.max_send_message_length", _MAX_MSG), ("grpc.max_receive_message_length", _MAX_MSG)]

  def _sync(self):
    import grpc
    if self._sync_channel is None:
      self._sync_channel = grpc.insecure_channel(self.target, options=self._opts())
    return self._sync_channel

  def _async(self):
    import grpc
    loop = asyncio.get_running_loop()
    ch = self._aio.get(id(loop))
    if ch is None:
      ch = grpc.aio.insecure_channel(self.target, options=self._opts())
      self._aio[id(loop)] = ch
    return ch

  def submit(self, method_name: Optional[str] = None, *args, **kwargs) -> Any:
    rpc = self._sync().unary_unary(f"/{_SERVICE}/Execute")
    payload = ExecutionRequest(method_name=method_name, args=args, kwargs=kwargs).serialize()
    return ExecutionResponse.deserialize(rpc(payload)).unwrap()

  async def asubmit(self, method_name: Optional[str] = None, *args, **kwargs) -> Any:
    rpc = self._async().unary_unary(f"/{_SERVICE}/Execute")
    payload = ExecutionRequest(method_name=method_name, args=args, kwargs=kwargs).serialize()
    return ExecutionResponse.deserialize(await rpc(payload)).unwrap()

  async def dispatch_task(self, request_id, method_name, *args, **kwargs) -> str:
    rpc = self._async().unary_unary(f"/{_SERVICE}/DispatchTask")
    return cloudpickle.loads(await rpc(ExecutionRequest(request_id, method_name, args, kwargs).serialize()))

  async def poll_responses(self, timeout_s: float = LONG_POLL_TIMEOUT_S, max_items: int = 64):
    rpc = self._async().unary_stream(f"/{_SERVICE}/PollResponses")
    out = []
    async for item in rpc(cloudpickle.dumps((timeout_s, max_items))):
      out.append(ExecutionResponse.deserialize(item))
    return out

  async def close(self) -> None:
    for ch in self._aio.values():
      await ch.close()
    self._aio.clear()
    if self._sync_channel is not None:
      self._sync_channel.close()
      self._sync_channel = None


RemoteActorHandle = GrpcRemoteActorHandle


# ---- pools --------------------------------------------------------------------------------------
class ActorPool(abc.ABC):
  @abc.abstractmethod
  def add_actor(self, actor: Union[str, ActorHandle]) -> None: ...

  @abc.abstractmethod
  def submit(self, method_name: Optional[str] = None, *args, **kwargs) -> Any: ...

  @abc.abstractmethod
  async def asubmit(self, method_name: Optional[str] = None, *args, **kwargs) -> Any: ...


TaskSpec = Tuple[str, str, Sequence[Any], Dict[str, Any]]       # (request_id, method, args, kwargs)


class RoutingActorPool(ActorPool):
  """Routing order: a custom `router` (callable, or object with a handler named after the
  method), else the `route_key` keyword (stable hash -> sticky actor; removed before the call),
  else `policy`: "round_robin" or "least_loaded" (fewest calls in flight through this pool)."""

  def __init__(self, actors: Optional[Sequence[Union[str, ActorHandle]]] = None, *, router: Any = None,
               policy: str = "round_robin"):
    if policy not in ("round_robin", "least_loaded"):
      raise ValueError(f"unknown routing policy {policy!r}")
    self._actors: List[ActorHandle] = []
    self._inflight: Dict[int, int] = {}
    self._idx = 0
    self.router, self.policy = router, policy
    for a in actors or []:
      self.add_actor(a)

  @property
  def actors(self) -> List[ActorHandle]:
    return list(self._actors)

  def add_actor(self, actor: Union[str, ActorHandle]) -> None:
    if isinstance(actor, str):
      actor = ActorHandle.from_address(actor)
    if not isinstance(actor, ActorHandle):
      raise TypeError(f"Expected str or ActorHandle, got {type(actor)}")
    self._actors.append(actor)
    self._inflight[id(actor)] = 0

  def _get_next_actor(self, method_name=None, args=(), kwargs=None) -> ActorHandle:
    if not self._actors:
      raise RuntimeError("RoutingActorPool contains no registered ActorHandles.")
    kwargs = kwargs or {}
    if self.router is not None:
      per_method = getattr(self.router, method_name, None) if method_name else None
      if callable(per_method):
        return per_method(self._actors, args, kwargs)
      if callable(self.router):
        return self.router(self._actors, method_name, args, kwargs)
      raise TypeError(f"Router object {type(self.router)} must provide a method matching '{method_name}' or be "
                      "callable.")
    key = kwargs.get("route_key")
    if key is not None:      # CRC of the key's text: the same key finds the same actor in every process and run
      return self._actors[zlib.crc32(repr(key).encode("utf-8")) % len(self._actors)]
    if self.policy == "least_loaded":
      return min(self._actors, key=lambda a: self._inflight[id(a)])
    actor = self._actors[self._idx % len(self._actors)]
    self._idx += 1
    return actor

  def submit(self, method_name: Optional[str] = None, *args, **kwargs) -> Any:
    actor = self._get_next_actor(method_name, args, kwargs)
    kwargs.pop("route_key", None)
    self._inflight[id(actor)] += 1
    try:
      return actor.submit(method_name, *args, **kwargs)
    finally:
      self._inflight[id(actor)] -= 1

  async def asubmit(self, method_name: Optional[str] = None, *args, **kwargs) -> Any:
    actor = self._get_next_actor(method_name, args, kwargs)
    kwargs.pop("route_key", None)
    self._inflight[id(actor)] += 1
    try:
      return await actor.asubmit(method_name, *args, **kwargs)
    finally:
      self._inflight[id(actor)] -= 1

  async def as_completed_stream(self, tasks: Sequence[TaskSpec]) -> AsyncIterator[Any]:
    """One-shot batch: yields results as they finish; the first failure is re-raised and the
    rest is abandoned."""
    if not self._actors:
      raise RuntimeError("RoutingActorPool contains no registered ActorHandles.")
    if not tasks:
      return
    async with self.execution_session(tasks) as session:
      async for result, exc in session.as_completed():
        if exc is not None:
          raise exc
        yield result

  @contextlib.asynccontextmanager
  async def execution_session(self, initial_tasks: Optional[Sequence[TaskSpec]] = None):
    session = PoolExecutionSession(self)
    try:
      for rid, method, args, kwargs in initial_tasks or []:
        await session.submit(rid, method, *args, **kwargs)
      yield session
    finally:
      await session.close()


class PoolExecutionSession:
  """Dynamic, fault-isolated streaming over a pool: `submit` dispatches a task to a routed actor,
  one poller per actor collects finished responses, `as_completed` yields `(result, exception)`
  pairs until nothing is in flight; new tasks may be submitted while iterating."""

  def __init__(self, pool: RoutingActorPool):
    self._pool = pool
    self._done: asyncio.Queue = asyncio.Queue()
    self._in_flight = 0
    self._pollers: Dict[int, asyncio.Task] = {}
    self._pending_by_actor: Dict[int, int] = {}
    self._closed = False

  async def submit(self, request_id: Optional[str], method_name: str, *args, **kwargs) -> str:
    if self._closed:
      raise RuntimeError("session is closed")
    actor = self._pool._get_next_actor(method_name, args, kwargs)
    kwargs.pop("route_key", None)
    self._in_flight += 1
    self._pending_by_actor[id(actor)] = self._pending_by_actor.get(id(actor), 0) + 1
    self._pool._inflight[id(actor)] += 1
    try:
      rid = await actor.dispatch_task(request_id, method_name, *args, **kwargs)
    except BaseException:
      self._in_flight -= 1
      self._pending_by_actor[id(actor)] -= 1
      self._pool._inflight[id(actor)] -= 1
      raise
    if id(actor) not in self._pollers or self._pollers[id(actor)].done():
      self._pollers[id(actor)] = asyncio.create_task(self._poll(actor))
    return rid

  async def _poll(self, actor: ActorHandle) -> None:
    while not self._closed and self._pending_by_actor.get(id(actor), 0) > 0:
      try:
        responses = await actor.poll_responses(timeout_s=1.0)
      except asyncio.CancelledError:
        raise
      except Exception as e:                 # the transport failed: everything pending there is lost
        n = self._pending_by_actor.get(id(actor), 0)
        self._pending_by_actor[id(actor)] = 0
        self._pool._inflight[id(actor)] -= n
        for _ in range(n):
          await self._done.put((None, e))
        return
      for r in responses:
        self._pending_by_actor[id(actor)] -= 1
        self._pool._inflight[id(actor)] -= 1
        try:
          await self._done.put((r.unwrap(), None))
        except RuntimeError as e:
          await self._done.put((None, e))

  async def as_completed(self) -> AsyncIterator[Tuple[Any, Optional[BaseException]]]:
    while self._in_flight > 0:
      item = await self._done.get()
      self._in_flight -= 1
      yield item

  async def close(self) -> None:
    self._closed = True
    for t in self._pollers.values():
      t.cancel()
    for t in self._pollers.values():
      with contextlib.suppress(asyncio.CancelledError, Exception):
        await t


# ---- decorator ----------------------------------------------------------------------------------
def remote(cls_or_func: Any = None, *, transport: str = "inprocess", address: Optional[str] = None) -> Any:
  """`@remote class W: ...` -> `W.remote(*a, **k)` returns an `ActorHandle` (in-process instance,
  or a client of `address` for `transport="grpc"` / `@remote("grpc://host:port")`).
  `@remote def f(...)` -> `f.remote(...)` runs through an in-process handle."""
  if isinstance(cls_or_func, str):
    address, cls_or_func = cls_or_func, None
  if address and "://" in address and transport == "inprocess":
    transport = address.split("://")[0]

  def decorate(target: Any) -> Any:
    if inspect.isclass(target):
      class ActorFactory:
        @classmethod
        def remote(cls, *args, **kwargs) -> ActorHandle:
          if transport == "inprocess":
            return InProcessActorHandle(InProcessRemoteExecutionServer(target(*args, **kwargs)))
          if transport == "grpc":
            return ActorHandle.from_address(address or kwargs.pop("address", "grpc://localhost:50051"))
          raise ValueError(f"Unsupported transport: {transport}")
      ActorFactory.__name__, ActorFactory.__doc__ = target.__name__, target.__doc__
      ActorFactory.__wrapped__ = target
      return ActorFactory
    if inspect.isfunction(target) or inspect.ismethod(target):
      if transport != "inprocess":
        raise NotImplementedError(f"Remote execution over transport='{transport}' is not yet supported for "
                                  "standalone functions; decorate a class instead.")

      class _Holder:
        execute = staticmethod(target)
      handle = InProcessActorHandle(InProcessRemoteExecutionServer(_Holder()))

      def call(*args, **kwargs):
        if inspect.iscoroutinefunction(target):
          try:
            asyncio.get_running_loop()
            return handle.asubmit("execute", *args, **kwargs)
          except RuntimeError:
            pass
        return handle.submit("execute", *args, **kwargs)
      call.remote = call
      call.__name__, call.__doc__ = target.__name__, target.__doc__
      return call
    raise TypeError(f"@remote expects a class or function, got {type(target)}")

  return decorate if cls_or_func is None else decorate(cls_or_func)
