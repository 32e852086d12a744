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

import dataclasses
from typing import Any, Dict, Mapping, Optional

from ....rl.agentic.environments import base_environment
from ...rl.agentic import registry

# What each command can see. A node whose name ends in 3 has a GPU fault that only a GPU query shows.
_VISIBILITY = {"uptime": lambda node: "OK",
               "nvidia-smi --query-gpu=ecc.errors": lambda node: _true_state(node)}
_PLAYBOOK = {"easy": "uptime", "medium": "uptime", "hard": "nvidia-smi --query-gpu=ecc.errors"}


@dataclasses.dataclass
class ClusterClient:
  """Connection to a (pretend) cluster API: stateful, process-bound, unpicklable on purpose."""
  endpoint: str = "cluster.local"
  connected: bool = True
  commands: int = 0

  def run(self, node: str, command: str) -> str:
    if not self.connected:
      raise RuntimeError("cluster client is disconnected")
    self.commands += 1
    return f"[{node}] `{command}` -> {_VISIBILITY.get(command, _sees_nothing)(node)}"

  def close(self) -> None:
    self.connected = False

  def __reduce__(self):
    raise TypeError("ClusterClient holds a live connection and cannot be pickled")


def _sees_nothing(node: str) -> str:
  return "OK"


def _true_state(node: str) -> str:
  return "DEGRADED" if node.endswith("3") else "OK"


class _ClusterEpisode(base_environment.BaseTaskEnv):
  """One command against one node: reward 1 when the command reports the node's true state, 0 when it calls a
  faulty node healthy."""

  client: ClusterClient
  node: str

  def _initial_observation(self) -> Dict[str, Any]:
    return {"observation": f"Connected to {self.node}. Ready for commands."}

  def _step_impl(self, action: Any) -> base_environment.EnvStepResult:
    report = self.client.run(self.node, str(action))
    seen = report.rsplit(" ", 1)[-1]
    return base_environment.EnvStepResult(observation=report, reward=float(seen == _true_state(self.node)), done=True,
                                          info={"node": self.node, "degraded": seen == "DEGRADED"})

  def close(self) -> None:
    self.client.close()


@registry.register_env("cluster")
class ClusterTaskEnv(_ClusterEpisode):
  """Registered under "cluster": the episode plus a client built here, inside the worker process."""

  def __init__(self, task: Optional[Mapping[str, Any]] = None, **kwargs):
    task = dict(task or {})
    super().__init__(task=task, **kwargs)
    self.node, self.client = task.get("node", "node-0"), ClusterClient()


@registry.register_agent("triage")
@dataclasses.dataclass
class TriageAgent:
  """Picks a command from a playbook keyed by the task's difficulty (a real agent would ask the policy model)."""
  system_prompt: str = ""

  def step(self, observation: Any, difficulty: str = "easy") -> str:
    return _PLAYBOOK.get(difficulty, _PLAYBOOK["easy"])
