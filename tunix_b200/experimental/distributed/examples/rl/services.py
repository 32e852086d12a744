"""The two services of the toy RL system and how the orchestrator reaches them.

The reference generates gRPC stubs from a .proto for these (tunix/experimental/distributed/examples/rl/service.proto);
here a service is a plain object served by `GrpcRemoteExecutionServer`, and its client is an `ActorHandle`, so there is
nothing to generate. What a worker announces through discovery is one line of JSON (`announce` / `parse_announcement`).
"""
from __future__ import annotations

import ast
import json
import operator
import random
from typing import Any, Dict

from ....worker import remote_execution

_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul}


def evaluate(expression: str) -> int:
  """'3 + 4' -> 7 for + - * on integers; anything else is refused (prompts come over the network)."""
  node = ast.parse(expression.strip(), mode="eval").body
  if not (isinstance(node, ast.BinOp) and type(node.op) in _OPS and isinstance(node.left, ast.Constant)
          and isinstance(node.right, ast.Constant) and isinstance(node.left.value, int)
          and isinstance(node.right.value, int)):
    raise ValueError(f"not a simple integer expression: {expression!r}")
  return _OPS[type(node.op)](node.left.value, node.right.value)


class RolloutService:
  """'Generates' an answer to an arithmetic prompt that is off by -1, 0 or +1: a policy that is sometimes wrong."""

  def __init__(self, server_id: str, seed: int = 0):
    self.server_id, self._rng, self.served = server_id, random.Random(seed), 0

  def generate(self, prompt: str) -> str:
    self.served += 1
    return f"= {evaluate(prompt) + self._rng.randint(-1, 1)}"


class TrainerService:
  """Keeps a one-number 'model': the running accuracy of the completions it was trained on."""

  def __init__(self):
    self.steps, self.correct = 0, 0

  def train(self, prompt: str, completion: str) -> str:
    self.steps += 1
    self.correct += int(completion.strip() == f"= {evaluate(prompt)}")
    return f"step {self.steps}: accuracy {self.correct / self.steps:.2f}"


def serve(instance: Any, port: int, host: str = "127.0.0.1") -> remote_execution.GrpcRemoteExecutionServer:
  server = remote_execution.GrpcRemoteExecutionServer(instance)
  server.start_serving(port, host)
  return server


def announce(service_type: str, server_port: int, server_id: str = "") -> bytes:
  return json.dumps({"service_type": service_type, "server_port": int(server_port), "server_id": server_id}).encode()


def parse_announcement(metadata: bytes) -> Dict[str, Any]:
  info = json.loads(metadata.decode("utf-8"))
  if info.get("service_type") not in ("rollout", "trainer"):
    raise ValueError(f"unknown service type {info.get('service_type')!r}")
  return info
