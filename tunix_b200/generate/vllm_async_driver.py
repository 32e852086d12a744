"""Step-level driver of an in-process vLLM engine (tunix/generate/vllm_async_driver.py:53-409).

`LLM.generate` is a blocking batch call: requests that arrive while a batch is running wait for all of it. Agentic
rollouts produce requests one by one, at their own pace, and want each answer as soon as it is finished. This driver
owns the engine on one thread and works at the granularity of `engine.step()`:

  * `submit()` returns a `concurrent.futures.Future` at once; the request joins a waiting room;
  * the waiting room opens when `submission_threshold` requests wait or the oldest has waited `submission_timeout_s`
    (0 / 0 = every request goes in as it comes): this is what lets many episodes share the engine's batch;
  * admitted requests are handed to `engine.add_request`, then the thread calls `engine.step()` for as long as the
    engine has unfinished requests; a finished output resolves its future, an unfinished one goes to the optional
    `stream_callback`;
  * `cancel(request_id)` works in either place (waiting room: dropped; engine: `abort_request`), and the future is
    cancelled;
  * `pause()` stops stepping after the current step (weights are about to change) without losing requests;
    `resume()` continues; `shutdown()` cancels everything that has not finished.

An exception out of the engine fails every request in flight with that exception and is kept in `last_error`;
the driver keeps serving new requests afterwards.

The engine is duck-typed (`add_request(request_id, prompt, params)`, `step() -> outputs with .request_id and
.finished`, `has_unfinished_requests()`, `abort_request([ids])`), which is vLLM's `LLMEngine` surface; tests drive a
small fake with the same four methods.
"""
from __future__ import annotations

import collections
import concurrent.futures
import itertools
import threading
import time
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

StreamCallback = Callable[[Any], None]


class _Waiting:
  __slots__ = ("request_id", "prompt", "params", "future", "since")

  def __init__(self, request_id: str, prompt: Any, params: Any, future: concurrent.futures.Future):
    self.request_id, self.prompt, self.params, self.future = request_id, prompt, params, future
    self.since = time.monotonic()


class VLLMInProcessDriver:

  def __init__(self, llm_engine: Any, *, submission_threshold: int = 0, submission_timeout_s: float = 0.0,
               stream_callback: Optional[StreamCallback] = None, idle_wait_s: float = 0.05, auto_start: bool = True):
    if submission_threshold < 0 or submission_timeout_s < 0:
      raise ValueError("submission_threshold and submission_timeout_s must be >= 0")
    self._engine = llm_engine
    self._threshold, self._timeout = int(submission_threshold), float(submission_timeout_s)
    self._stream = stream_callback
    self._idle_wait = float(idle_wait_s)
    self._cv = threading.Condition()
    self._room: "collections.OrderedDict[str, _Waiting]" = collections.OrderedDict()    # not yet in the engine
    self._running: Dict[str, concurrent.futures.Future] = {}                              # in the engine
    self._abort: List[str] = []              # ids to abort inside the engine, applied by the engine thread
    self._paused = False
    self._stopping = False
    self._ids = itertools.count()
    self._thread: Optional[threading.Thread] = None
    self.last_error: Optional[BaseException] = None
    self.steps = 0
    if auto_start:
      self.start()

  @classmethod
  def from_llm(cls, llm: Any, **kwargs) -> "VLLMInProcessDriver":
    """From a `vllm.LLM`: its engine is `llm.llm_engine`."""
    return cls(llm.llm_engine, **kwargs)

  @property
  def llm_engine(self) -> Any:
    return self._engine

  # ---- client side -----------------------------------------------------------------------------
  def start(self) -> None:
    with self._cv:
      if self._thread is not None and self._thread.is_alive():
        return
      self._stopping = False
      self._thread = threading.Thread(target=self._serve, daemon=True, name="vllm-step-driver")
      self._thread.start()

  def submit(self, prompt: Any, params: Any, request_id: Optional[str] = None) -> concurrent.futures.Future:
    """`prompt` is whatever the engine's `add_request` takes (e.g. {"prompt_token_ids": [...]})."""
    future: concurrent.futures.Future = concurrent.futures.Future()
    with self._cv:
      if self._stopping:
        raise RuntimeError("driver is shut down")
      rid = request_id if request_id is not None else f"req-{next(self._ids)}"
      if rid in self._room or rid in self._running:
        raise ValueError(f"request id {rid!r} is already in flight")
      future.request_id = rid                      # callers cancel by this id
      self._room[rid] = _Waiting(rid, prompt, params, future)
      self._cv.notify_all()
    return future

  submit_request = submit

  def submit_requests(self, prompts: Sequence[Any], params: Any) -> List[concurrent.futures.Future]:
    """One future per prompt; `params` is shared or a sequence of the same length."""
    each = params if isinstance(params, (list, tuple)) else [params] * len(prompts)
    if len(each) != len(prompts):
      raise ValueError("one sampling-params object per prompt, or one for all")
    return [self.submit(p, sp) for p, sp in zip(prompts, each)]

  def cancel(self, request_id: str) -> bool:
    """True when the request was still in flight."""
    with self._cv:
      waiting = self._room.pop(request_id, None)
      if waiting is not None:
        waiting.future.cancel()
        return True
      future = self._running.pop(request_id, None)
      if future is None:
        return False
      self._abort.append(request_id)
      future.cancel()
      self._cv.notify_all()
      return True

  def pause(self) -> None:
    """Returns when the engine thread is between steps and will not start another one."""
    with self._cv:
      self._paused = True
      self._cv.notify_all()
      self._cv.wait_for(lambda: not self._stepping)

  def resume(self) -> None:
    with self._cv:
      self._paused = False
      self._cv.notify_all()

  def shutdown(self, timeout: float = 5.0) -> None:
    with self._cv:
      self._stopping = True
      self._cv.notify_all()
    if self._thread is not None:
      self._thread.join(timeout)
    with self._cv:
      for waiting in self._room.values():
        waiting.future.cancel()
      for future in self._running.values():
        future.cancel()
      self._room.clear()
      self._running.clear()

  stop = shutdown

  def __enter__(self) -> "VLLMInProcessDriver":
    return self

  def __exit__(self, *exc) -> None:
    self.shutdown()

  @property
  def in_flight(self) -> Tuple[int, int]:
    """(waiting, running)."""
    with self._cv:
      return len(self._room), len(self._running)

  # ---- engine thread ---------------------------------------------------------------------------
  _stepping = False

  def _room_is_open(self) -> bool:
    if not self._room:
      return False
    if self._threshold <= 1 and self._timeout == 0.0:
      return True
    if self._threshold and len(self._room) >= self._threshold:
      return True
    oldest = next(iter(self._room.values())).since
    return time.monotonic() - oldest >= self._timeout

  def _next_wake(self) -> float:
    """Seconds until the waiting room would open by age (idle wait when nothing waits)."""
    if not self._room or self._room_is_open():
      return self._idle_wait
    oldest = next(iter(self._room.values())).since
    return max(0.0, min(self._idle_wait, self._timeout - (time.monotonic() - oldest)))

  def _serve(self) -> None:
    while True:
      with self._cv:
        while not self._stopping and (self._paused or not (self._running or self._abort or self._room_is_open())):
          self._cv.wait(self._next_wake())
        if self._stopping:
          return
        admitted = list(self._room.values()) if self._room_is_open() else []
        for w in admitted:
          del self._room[w.request_id]
          self._running[w.request_id] = w.future
        aborts, self._abort = self._abort, []
        self._stepping = True
      try:
        outputs = self._advance(admitted, aborts)
      except BaseException as e:  # noqa: BLE001 - reported through the futures
        self._fail_all(e)
        outputs = []
      finished = []
      with self._cv:
        for out in outputs:
          rid = getattr(out, "request_id", None)
          if getattr(out, "finished", True):
            future = self._running.pop(rid, None)
            if future is not None:
              finished.append((future, out))
          elif self._stream is not None and rid in self._running:
            finished.append((None, out))
        self._stepping = False
        self._cv.notify_all()
      for future, out in finished:          # callbacks run outside the lock
        if future is None:
          self._stream(out)
        else:
          _settle(future, result=out)

  def _advance(self, admitted: Iterable[_Waiting], aborts: List[str]) -> List[Any]:
    if aborts:
      self._engine.abort_request(aborts)
    for w in admitted:
      self._engine.add_request(w.request_id, w.prompt, w.params)
    if not self._engine.has_unfinished_requests():
      return []
    self.steps += 1
    return list(self._engine.step())

  def _fail_all(self, error: BaseException) -> None:
    self.last_error = error
    with self._cv:
      failed, self._running = list(self._running.items()), {}
    try:
      self._engine.abort_request([rid for rid, _ in failed])
    except Exception:  # noqa: BLE001 - the engine is already in trouble
      pass
    for _, future in failed:
      _settle(future, error=error)


def _settle(future: concurrent.futures.Future, result: Any = None, error: Optional[BaseException] = None) -> None:
  """Futures stay PENDING until they are settled, so that `cancel()` works at any time before; a cancellation
  that wins the race makes the late result a no-op."""
  try:
    if error is not None:
      future.set_exception(error)
    else:
      future.set_result(result)
  except concurrent.futures.InvalidStateError:
    pass
