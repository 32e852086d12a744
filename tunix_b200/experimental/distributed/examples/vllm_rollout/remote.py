"""Remote method invocation in one page: a server and a client in the same event loop
(tunix/experimental/distributed/examples/vllm_rollout/remote.py).

  python -m tunix_b200.experimental.distributed.runtime.main \\
      --process_main=tunix_b200.experimental.distributed.examples.vllm_rollout.remote.main

The server binds a plain object; the client holds an `ActorHandle` to its address and calls methods by name, once
awaiting the result (`asubmit`) and once in fire-and-collect style (`dispatch_task` / `poll_responses`), which is
how long generations are driven without holding a connection open per request.
"""
from __future__ import annotations

import asyncio
import os
from typing import Any, Dict, List

from ....worker import remote_execution


class Worker:
  """What gets served: any object; methods may be plain or coroutines."""

  def get_worker_id(self) -> str:
    return f"worker-{os.getpid()}"

  async def slow_square(self, x: int, delay_s: float = 0.01) -> int:
    await asyncio.sleep(delay_s)
    return x * x


async def run_loop() -> Dict[str, Any]:
  server = remote_execution.GrpcRemoteExecutionServer(Worker())
  await server.start_serving_async(port=0)
  handle = remote_execution.ActorHandle.from_address(f"grpc://127.0.0.1:{server.port}")
  try:
    worker_id = await handle.asubmit("get_worker_id")
    for x in (3, 4, 5):
      await handle.dispatch_task(f"square-{x}", "slow_square", x)
    squares: List[int] = []
    while len(squares) < 3:
      squares += [r.unwrap() for r in await handle.poll_responses(timeout_s=5.0)]
    return {"worker_id": worker_id, "squares": sorted(squares)}
  finally:
    await handle.close()
    await server.stop_serving()


def main(ctx, argv) -> Dict[str, Any]:
  result = asyncio.run(run_loop())
  print(result)
  return result
