"""An agent and an environment that register themselves by name
(tunix/experimental/worker/examples/sample_agent_and_env.py).

A rollout request travels between processes, so it can only carry plain data: it names the agent and environment
types ("triage", "cluster") and the task, and the worker builds the objects where they will live.
`registry.auto_discover_modules("tunix_b200.experimental.worker.examples")` finds this file by its decorators and
imports it, which fills the registries.

The environment owns a `ClusterClient`, a stand-in for a client library that holds sockets and credentials (a
Kubernetes or Slurm client): it refuses to be pickled, which is exactly why it has to be created on the worker.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

from ....rl.agentic.environments import base_environment
from ...rl.agentic import registry


class ClusterClient:
  """Connection to a (pretend) cluster API. Stateful and process-bound."""

  def __init__(self, endpoint: str = "cluster.local"):
    self.endpoint, self.connected, self.commands = endpoint, True, 0

  def run(self, node: str, command: str) -> str:
    if not self.connected:
      raise RuntimeError("cluster client is disconnected")
    self.commands += 1
    status = "DEGRADED" if "gpu" in command and node.endswith("3") else "OK"
    return f"[{node}] `{command}` -> {status}"

  def close(self) -> None:
    self.connected = False

  def __reduce__(self):
    raise TypeError("ClusterClient holds a live connection and cannot be pickled")


@registry.register_env("cluster")
class ClusterTaskEnv(base_environment.BaseTaskEnv):
  """One command against one node. Nodes whose name ends in 3 have a GPU fault that only a GPU query shows: the
  reward is 1 when the command reports the node's true state, 0 when it calls a faulty node healthy."""

  def __init__(self, task: Optional[Dict[str, Any]] = None, **kwargs):
    super().__init__(task=task, **kwargs)
    self.client = ClusterClient()                       # built here, inside the worker process
    self.node = (task or {}).get("node", "node-0")

  def _initial_observation(self) -> Dict[str, Any]:
    return {"observation": f"Connected to {self.node}. Ready for commands."}

  def _step_impl(self, action: Any) -> base_environment.EnvStepResult:
    result = self.client.run(self.node, str(action))
    found_fault = result.endswith("DEGRADED")
    missed_fault = self.node.endswith("3") and not found_fault
    return base_environment.EnvStepResult(observation=result, reward=0.0 if missed_fault else 1.0, done=True,
                                          info={"node": self.node, "degraded": found_fault})

  def close(self) -> None:
    self.client.close()


@registry.register_agent("triage")
class TriageAgent:
  """Chooses what to run from the task's difficulty (a real agent would ask the policy model)."""

  def __init__(self, system_prompt: str = ""):
    self.system_prompt = system_prompt

  def step(self, observation: Any, difficulty: str = "easy") -> str:
    return "nvidia-smi --query-gpu=ecc.errors" if difficulty == "hard" else "uptime"
