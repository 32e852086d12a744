"""One rollout request served by a worker in another server, with the agent and environment built on the worker
(tunix/experimental/worker/examples/agentic_remote_execution_demo.py).

  python -m tunix_b200.experimental.worker.examples.agentic_remote_execution_demo

The orchestrator side holds an `ActorHandle` and sends a `RolloutRequest` whose metadata names the agent type, the
environment type and the task. The worker side (`RegistryRolloutWorker`) looks both up in the registries, runs the
episode and answers with a `RolloutResponse`. Nothing but plain data crosses the wire; the environment's client
object, which cannot be pickled, never leaves the worker.
"""
from __future__ import annotations

import asyncio
import logging
import random
from typing import Any, Dict, Optional, Tuple

from ...common import datatypes
from ...rl.agentic import registry
from .. import abstract_worker, remote_execution

EXAMPLES_PACKAGE = "tunix_b200.experimental.worker.examples"
WorkerState = datatypes.WorkerState


class RegistryRolloutWorker(abstract_worker.Worker):
  """A rollout worker whose agents and environments come from the registries, per request."""

  def __init__(self, worker_id: str, min_delay_s: float = 0.0, max_delay_s: float = 0.0, seed: int = 0):
    self.worker_id = worker_id
    self._delay = (min_delay_s, max_delay_s)
    self._rng = random.Random(seed)
    self._state = WorkerState.PENDING
    self.policy_version = 0
    self.served = 0

  # ---- lifecycle
  def initialize(self) -> datatypes.Response:
    with self._phase(WorkerState.INITIALIZING):
      registry.auto_discover_modules(EXAMPLES_PACKAGE)
    return datatypes.Response(metadata={"agents": registry.AGENT_REGISTRY.keys(), "envs": registry.ENV_REGISTRY.keys()})

  def compile(self, dummy_data: Any = None) -> datatypes.Response:
    return datatypes.Response()

  def start(self) -> datatypes.Response:
    return datatypes.Response()

  def stop(self) -> datatypes.Response:
    self._state = WorkerState.STOPPED
    return datatypes.Response()

  def info(self) -> datatypes.WorkerInfo:
    return datatypes.WorkerInfo(worker_id=self.worker_id, roles=frozenset({"rollout"}), resources={})

  def heartbeat(self) -> datatypes.HealthReport:
    return datatypes.HealthReport(state=self.state, policy_version=self.policy_version)

  # ---- serving
  def _build(self, metadata: Dict[str, Any], task: Dict[str, Any]) -> Tuple[Any, Any]:
    agent_cls = registry.AGENT_REGISTRY.get(metadata.get("agent_type", "triage"))
    env_cls = registry.ENV_REGISTRY.get(metadata.get("env_type", "cluster"))
    return agent_cls(system_prompt=metadata.get("system_prompt", "")), env_cls(task=task)

  async def generate(self, request: datatypes.RolloutRequest) -> datatypes.RolloutResponse:
    if self.state == WorkerState.PENDING:
      self.initialize()
    task = request.prompt if isinstance(request.prompt, dict) else {"prompt": request.prompt}
    task = {**task, **{k: v for k, v in request.metadata.items() if k in ("node", "difficulty")}}
    low, high = self._delay
    if high > 0:
      await asyncio.sleep(self._rng.uniform(low, high))        # episodes finish out of order
    agent, env = self._build(request.metadata, task)
    try:
      observation, _ = env.reset()
      action = agent.step(observation, difficulty=task.get("difficulty", "easy"))
      result = env.step(action)
      observation, reward = result[0], float(result[1])
    finally:
      env.close()
    self.served += 1
    return datatypes.RolloutResponse(
        request_id=request.request_id, prompt_id=request.prompt_id, status="SUCCEEDED", env_reward=reward,
        policy_version=self.policy_version,
        metadata={"worker_id": self.worker_id, "action": action, "observation": str(observation),
                  "policy_version": self.policy_version})

  def sync_weights(self, policy_version: int) -> datatypes.Response:
    self.policy_version = int(policy_version)
    return datatypes.Response(metadata={"worker_id": self.worker_id, "policy_version": self.policy_version})


async def start_rollout_server(port: int = 0, worker_id: str = "rollout-worker-1", **worker_kwargs
                               ) -> remote_execution.GrpcRemoteExecutionServer:
  """Serves a `RegistryRolloutWorker` on `port` (0: any free port, see `server.port`) from the running loop."""
  server = remote_execution.GrpcRemoteExecutionServer(RegistryRolloutWorker(worker_id, **worker_kwargs))
  await server.start_serving_async(port=port)
  return server


async def run_orchestrator_node(address: str, node: str = "node-13", difficulty: str = "hard",
                                request_id: str = "req-1") -> datatypes.RolloutResponse:
  handle = remote_execution.ActorHandle.from_address(address)
  try:
    await handle.asubmit("initialize")
    request = datatypes.RolloutRequest(
        request_id=request_id, prompt_id="p-1", prompt={"prompt": f"Find out what is wrong with {node}"},
        metadata={"agent_type": "triage", "env_type": "cluster", "node": node, "difficulty": difficulty,
                  "system_prompt": "You are a cluster on-call engineer."})
    return await handle.asubmit("generate", request)
  finally:
    await handle.close()


async def demo() -> datatypes.RolloutResponse:
  server = await start_rollout_server()
  try:
    response = await run_orchestrator_node(f"grpc://127.0.0.1:{server.port}")
  finally:
    await server.stop_serving()
  logging.info("worker %s ran `%s` -> %s (reward %.1f)", response.metadata["worker_id"], response.metadata["action"],
               response.metadata["observation"], response.env_reward)
  return response


if __name__ == "__main__":
  logging.basicConfig(level=logging.INFO, format="%(message)s")
  asyncio.run(demo())
