"""A whole RL data loop over a pool of remote rollout workers
(tunix/experimental/worker/examples/rl_loop_remote_execution_demo.py).

  python -m tunix_b200.experimental.worker.examples.rl_loop_remote_execution_demo --workers 3 --epochs 2

Per epoch: every prompt of the batch becomes a `RolloutRequest` submitted to a `RoutingActorPool` session; the
results stream back in completion order (episodes take different times on different workers), a failed request
costs that request only, and when the batch is done the new policy version is pushed to every worker before the
next epoch. Training itself is left out: the point is the traffic.
"""
from __future__ import annotations

import argparse
import asyncio
import logging
import random
from typing import Any, Dict, List, Sequence

from ...common import datatypes
from .. import remote_execution
from . import agentic_remote_execution_demo as worker_demo


def synthetic_prompt_batches(num_batches: int = 3, batch_size: int = 4, seed: int = 0) -> List[List[Dict[str, Any]]]:
  rng = random.Random(seed)
  return [[{"prompt_id": f"prompt_b{b}_i{i}", "prompt": f"Check node-{b}{i}", "node": f"node-{b}{i}",
            "difficulty": rng.choice(["easy", "medium", "hard"]), "agent_type": "triage", "env_type": "cluster"}
           for i in range(batch_size)] for b in range(num_batches)]


def _request(epoch: int, index: int, item: Dict[str, Any], policy_version: int) -> datatypes.RolloutRequest:
  return datatypes.RolloutRequest(
      request_id=f"epoch_{epoch}_req_{index}", prompt_id=item["prompt_id"], prompt={"prompt": item["prompt"]},
      target_policy_version=policy_version,
      metadata={k: item[k] for k in ("agent_type", "env_type", "difficulty", "node")})


async def run_rl_training_loop(worker_addresses: Sequence[Any], num_epochs: int = 2, batch_size: int = 4,
                               seed: int = 0) -> List[Dict[str, Any]]:
  """`worker_addresses`: "grpc://host:port" strings or ready `ActorHandle`s. Returns one metrics dict per epoch."""
  pool = remote_execution.RoutingActorPool(list(worker_addresses))
  policy_version = 1
  for actor in pool.actors:
    await actor.asubmit("sync_weights", policy_version)
  report: List[Dict[str, Any]] = []
  for epoch, batch in enumerate(synthetic_prompt_batches(num_epochs, batch_size, seed)):
    done: List[datatypes.RolloutResponse] = []
    failed = 0
    async with pool.execution_session() as session:
      for index, item in enumerate(batch):
        await session.submit(f"epoch_{epoch}_req_{index}", "generate", _request(epoch, index, item, policy_version))
      async for result, error in session.as_completed():
        if error is not None:
          failed += 1
          logging.warning("a rollout failed: %s", error)
          continue
        done.append(result)
        logging.info("  %s on %s: `%s` reward %.1f", result.request_id, result.metadata["worker_id"],
                     result.metadata["action"], result.env_reward)
    report.append({"epoch": epoch, "policy_version": policy_version, "completed": len(done), "failed": failed,
                   "avg_reward": sum(r.env_reward for r in done) / len(done) if done else 0.0,
                   "workers": sorted({r.metadata["worker_id"] for r in done}),
                   "stale": sum(r.policy_version != policy_version for r in done)})
    logging.info("epoch %d: %d completed, %d failed, mean reward %.3f", epoch, len(done), failed,
                 report[-1]["avg_reward"])
    policy_version += 1
    for actor in pool.actors:
      await actor.asubmit("sync_weights", policy_version)
  for actor in pool.actors:
    await actor.close()
  return report


async def demo(workers: int = 2, epochs: int = 2, batch_size: int = 4) -> List[Dict[str, Any]]:
  servers = [await worker_demo.start_rollout_server(worker_id=f"rollout-worker-{i}", min_delay_s=0.01,
                                                    max_delay_s=0.05, seed=i) for i in range(workers)]
  try:
    return await run_rl_training_loop([f"grpc://127.0.0.1:{s.port}" for s in servers], epochs, batch_size)
  finally:
    for s in servers:
      await s.stop_serving()


if __name__ == "__main__":
  p = argparse.ArgumentParser()
  p.add_argument("--workers", type=int, default=2)
  p.add_argument("--epochs", type=int, default=2)
  p.add_argument("--batch_size", type=int, default=4)
  a = p.parse_args()
  logging.basicConfig(level=logging.INFO, format="%(message)s")
  for row in asyncio.run(demo(a.workers, a.epochs, a.batch_size)):
    print(row)
