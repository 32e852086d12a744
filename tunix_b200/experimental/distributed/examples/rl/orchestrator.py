"""Orchestrator of the toy RL system (tunix/experimental/distributed/examples/rl/orchestrator.py).

It shows the data flow of a disaggregated RL job and nothing of an RL algorithm: workers find the orchestrator
through discovery, the orchestrator turns each announcement into a client handle, and then every iteration sends a
prompt to one of the rollout workers and the (prompt, completion) pair to the trainer.

  python -m tunix_b200.experimental.distributed.runtime.main \\
      --process --process_main=tunix_b200.experimental.distributed.examples.rl.orchestrator.main \\
                --discovery_id=orchestrator --discovery_port=12345 --max_train_step=20 \\
      --process --process_main=tunix_b200.experimental.distributed.examples.rl.rollout.main \\
                --discovery_id=rollout-a --discovery_addrs=orchestrator:12345 --server_id=a --server_port=11111 \\
      --process --process_main=tunix_b200.experimental.distributed.examples.rl.rollout.main \\
                --discovery_id=rollout-b --discovery_addrs=orchestrator:12345 --server_id=b --server_port=11112 \\
      --process --process_main=tunix_b200.experimental.distributed.examples.rl.trainer.main \\
                --discovery_id=trainer --discovery_addrs=orchestrator:12345 --server_port=22222

On Kubernetes the same three bodies run in three replicated jobs of a JobSet with `--process_executor=...K8sExecutor`;
the discovery id is then the job's name.
"""
import argparse
import logging
import random
import threading
from typing import Dict, List, Optional

from ....worker import remote_execution
from . import services
from .rollout import stop


class Directory:
  """Client handles by role, filled in by discovery callbacks, waited on by the main loop."""

  def __init__(self, resolve_host=lambda host: "127.0.0.1"):
    self._resolve = resolve_host
    self._cv = threading.Condition()
    self.rollouts: Dict[str, remote_execution.ActorHandle] = {}
    self.trainer: Optional[remote_execution.ActorHandle] = None

  def accept(self, hostname: str, discovery_port: int, metadata: bytes) -> None:
    info = services.parse_announcement(metadata)
    address = f"{self._resolve(hostname)}:{info['server_port']}"
    handle = remote_execution.ActorHandle.from_address(f"grpc://{address}")
    logging.info("discovered %s service %s at %s", info["service_type"], info["server_id"], address)
    with self._cv:
      if info["service_type"] == "rollout":
        self.rollouts[info["server_id"]] = handle
      else:
        self.trainer = handle
      self._cv.notify_all()

  def wait(self, min_rollouts: int, timeout_s: float) -> None:
    with self._cv:
      if not self._cv.wait_for(lambda: self.trainer is not None and len(self.rollouts) >= min_rollouts, timeout_s):
        raise SystemExit(f"after {timeout_s:.0f} s: {len(self.rollouts)} of {min_rollouts} rollout workers, "
                         f"trainer {'found' if self.trainer else 'missing'}")


def main(ctx, argv) -> List[str]:
  parser = argparse.ArgumentParser()
  parser.add_argument("--message", type=str, default="this is orchestrator!")
  parser.add_argument("--max_train_step", type=int, default=100)
  parser.add_argument("--min_rollouts", type=int, default=2)
  parser.add_argument("--wait_s", type=float, default=60.0)
  parser.add_argument("--seed", type=int, default=0)
  args = parser.parse_args(argv)
  logging.info(args.message)
  directory = Directory()
  ctx.ipc.discovery.on_register(directory.accept)
  directory.wait(args.min_rollouts, args.wait_s)
  rng = random.Random(args.seed)
  history: List[str] = []
  try:
    for step in range(args.max_train_step):
      prompt = f"{rng.randint(0, 10)} {rng.choice('+-*')} {rng.randint(0, 10)}"
      server_id = rng.choice(sorted(directory.rollouts))
      completion = directory.rollouts[server_id].submit("generate", prompt)
      weights = directory.trainer.submit("train", prompt, completion)
      history.append(f"[{step}] {prompt} -> [{server_id}] {completion} -> [trainer] {weights}")
      logging.info(history[-1])
  finally:
    stop.set()                     # the serving bodies of this launcher (if any) end with the orchestrator
  return history
