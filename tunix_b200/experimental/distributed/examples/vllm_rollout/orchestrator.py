"""Generation load over discovered rollout workers
(tunix/experimental/distributed/examples/vllm_rollout/orchestrator.py).

  python -m tunix_b200.experimental.distributed.runtime.main \\
      --process --process_main=tunix_b200.experimental.distributed.examples.vllm_rollout.orchestrator.main \\
                --discovery_id=orchestrator --discovery_port=12400 --num_requests=64 --concurrency=8 \\
      --process --process_main=tunix_b200.experimental.distributed.examples.vllm_rollout.rollout.main \\
                --discovery_id=rollout-a --discovery_addrs=orchestrator:12400 --worker_id=a --port=50081 \\
      --process --process_main=tunix_b200.experimental.distributed.examples.vllm_rollout.rollout.main \\
                --discovery_id=rollout-b --discovery_addrs=orchestrator:12400 --worker_id=b --port=50082

`concurrency` client threads each pick a worker at random and ask it for one completion, until `num_requests` are
done; a monitor counts requests and generated tokens per worker and logs a summary every few seconds and at the end.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import dataclasses
import logging
import random
import threading
import time
from typing import Any, Dict, List, Sequence

from ....common import datatypes
from ....worker import remote_execution
from . import rollout as rollout_body


@dataclasses.dataclass(frozen=True)
class RolloutSpec:
  worker_id: str
  address: str
  model_name: str

  @classmethod
  def from_announcement(cls, host: str, metadata: bytes) -> "RolloutSpec":
    worker_id, port, model = metadata.decode("utf-8").split("|")
    return cls(worker_id=worker_id, address=f"grpc://{host}:{int(port)}", model_name=model)


class RequestStatsMonitor:
  """Per-worker counters behind a lock; `maybe_log_summary` logs at most once per interval."""

  def __init__(self, log_interval_seconds: float = 10.0):
    self._interval = log_interval_seconds
    self._lock = threading.Lock()
    self._requests: Dict[str, int] = {}
    self._tokens: Dict[str, int] = {}
    self._started = self._last_log = time.monotonic()

  @property
  def total_requests(self) -> int:
    with self._lock:
      return sum(self._requests.values())

  def record_request(self, worker_id: str, tokens: int = 0) -> None:
    with self._lock:
      self._requests[worker_id] = self._requests.get(worker_id, 0) + 1
      self._tokens[worker_id] = self._tokens.get(worker_id, 0) + int(tokens)

  def summary(self) -> Dict[str, Any]:
    with self._lock:
      elapsed = max(time.monotonic() - self._started, 1e-9)
      return {"elapsed_s": elapsed, "requests": dict(self._requests), "tokens": dict(self._tokens),
              "requests_per_s": sum(self._requests.values()) / elapsed,
              "tokens_per_s": sum(self._tokens.values()) / elapsed}

  def maybe_log_summary(self, force: bool = False) -> bool:
    now = time.monotonic()
    with self._lock:
      due = force or now - self._last_log >= self._interval
      if due:
        self._last_log = now
    if due:
      s = self.summary()
      logging.info("%d requests in %.1f s (%.1f req/s, %.0f tok/s): %s", sum(s["requests"].values()), s["elapsed_s"],
                   s["requests_per_s"], s["tokens_per_s"], s["requests"])
    return due


def orchestrator_main(workers: Sequence[RolloutSpec], num_requests: int, concurrency: int, max_tokens: int,
                      seed: int = 0, monitor: RequestStatsMonitor = None) -> Dict[str, Any]:
  monitor = monitor or RequestStatsMonitor()
  handles = {w.worker_id: remote_execution.ActorHandle.from_address(w.address) for w in workers}
  rng, rng_lock = random.Random(seed), threading.Lock()
  failures: List[str] = []

  def one_request(index: int) -> None:
    with rng_lock:
      spec = rng.choice(list(workers))
      a, b = rng.randint(0, 99), rng.randint(0, 99)
    request = datatypes.RolloutRequest(request_id=f"load-{index}", prompt_id=f"load-{index}", prompt=f"{a} + {b} =",
                                       generation_kwargs={"max_tokens": max_tokens, "temperature": 1.0, "seed": index})
    try:
      (response,) = handles[spec.worker_id].submit("generate", requests=[request])
      if response.status != "SUCCEEDED":
        raise RuntimeError(f"{response.status}: {response.error.message if response.error else ''}")
      monitor.record_request(spec.worker_id, sum(len(s.tokens) for s in response.segments))
    except Exception as e:  # noqa: BLE001 - a failed request is a line in the report
      failures.append(f"load-{index} on {spec.worker_id}: {e}")
    monitor.maybe_log_summary()
  with concurrent.futures.ThreadPoolExecutor(max_workers=max(1, concurrency)) as pool:
    list(pool.map(one_request, range(num_requests)))
  monitor.maybe_log_summary(force=True)
  return {**monitor.summary(), "failures": failures}


def main(ctx, argv) -> Dict[str, Any]:
  parser = argparse.ArgumentParser()
  parser.add_argument("--num_workers", type=int, default=2)
  parser.add_argument("--num_requests", type=int, default=64)
  parser.add_argument("--concurrency", type=int, default=8)
  parser.add_argument("--max_tokens", type=int, default=32)
  parser.add_argument("--wait_s", type=float, default=300.0)
  args = parser.parse_args(argv)
  found: List[RolloutSpec] = []
  enough = threading.Condition()

  def accept_worker(hostname: str, _port: int, metadata: bytes) -> None:
    spec = RolloutSpec.from_announcement("127.0.0.1", metadata)
    logging.info("discovered rollout worker %s (%s) at %s", spec.worker_id, spec.model_name, spec.address)
    with enough:
      found.append(spec)
      enough.notify_all()
  ctx.ipc.discovery.on_register(accept_worker)
  try:
    with enough:
      if not enough.wait_for(lambda: len(found) >= args.num_workers, args.wait_s):
        raise SystemExit(f"only {len(found)} of {args.num_workers} rollout workers announced themselves")
    return orchestrator_main(list(found), args.num_requests, args.concurrency, args.max_tokens)
  finally:
    rollout_body.stop.set()
