"""The control plane end to end with simulated workers, as a script or notebook cell
(tunix/experimental/orchestrator/simple_orchestrator_nb.py:28-156).

  python -m tunix_b200.experimental.orchestrator.simple_orchestrator_nb

No model anywhere: two rollout workers answer every request with a few made-up tokens (and count what they served),
one trainer worker records the batches it is given. What is real is everything between them - registration by role,
lifecycle, request expansion into groups, routing (samples of one prompt reach one worker), grouping of finished
rollouts, rewards, advantages, batch assembly and the training calls - so the printed table shows how data flows
through `ClusterOrchestrator.run` before any accelerator is involved.
"""
from __future__ import annotations

import zlib
from typing import Any, Dict, List, Optional, Sequence

import numpy as np

from ..common import datatypes
from ..worker import abstract_worker
from . import algorithm_adapter, batch_assembly, orchestrator as orchestrator_lib

WorkerState = datatypes.WorkerState


class _Simulated(abstract_worker.Worker):
  """Lifecycle of a worker that has nothing to load."""

  def __init__(self, worker_id: str, role: Any):
    self.worker_id, self._role = worker_id, role
    self._state = WorkerState.PENDING

  def info(self) -> datatypes.WorkerInfo:
    return datatypes.WorkerInfo(worker_id=self.worker_id, roles=frozenset({getattr(self._role, "value", self._role)}),
                                resources={"simulated": True})

  def initialize(self) -> datatypes.Response:
    with self._phase(WorkerState.INITIALIZING):
      pass
    return datatypes.Response()

  def compile(self, dummy_data: Any = None) -> datatypes.Response:
    with self._phase(WorkerState.COMPILING):
      pass
    return datatypes.Response()

  def start(self) -> datatypes.Response:
    return datatypes.Response()

  def stop(self) -> datatypes.Response:
    self._state = WorkerState.STOPPED
    return datatypes.Response()

  def heartbeat(self) -> datatypes.HealthReport:
    return datatypes.HealthReport(state=self.state)


class SimulatedRolloutWorker(_Simulated):
  """Completion tokens are a function of the prompt and the sample index, so runs repeat exactly; the completion
  length varies with the sample, which gives the length-based reward below something to rank."""

  def __init__(self, worker_id: str):
    super().__init__(worker_id, datatypes.Role.ROLLOUT)
    self.served: List[str] = []

  async def generate(self, requests: Optional[Sequence[datatypes.RolloutRequest]] = None,
                     prompts: Optional[Sequence[Any]] = None, **kwargs: Any) -> List[datatypes.RolloutResponse]:
    out = []
    for request in list(requests or []):
      seed = zlib.crc32(f"{request.prompt}|{request.group_offset_id}".encode())
      length = 2 + seed % 4
      tokens = np.asarray([20 + (seed >> (3 * i)) % 50 for i in range(length)], np.int32)
      prompt_tokens = np.asarray([10 + b % 40 for b in str(request.prompt).encode()[:6]], np.int32)
      self.served.append(request.request_id)
      out.append(datatypes.RolloutResponse(
          request_id=request.request_id, prompt_id=request.prompt_id, status="SUCCEEDED", prompt_tokens=prompt_tokens,
          segments=[datatypes.TokenSegment(source="assistant", tokens=tokens, loss_mask=np.ones(length, np.int32),
                                           logps=np.full(length, -1.0, np.float32))],
          policy_version=request.target_policy_version, metadata={**request.metadata, "worker_id": self.worker_id}))
    return out


class SimulatedTrainerWorker(_Simulated):
  """Records what it is asked to train on and reports a loss that falls with every optimizer step."""

  def __init__(self, worker_id: str, role: Any = datatypes.Role.ACTOR):
    super().__init__(worker_id, role)
    self.batches: List[Any] = []
    self.optimizer_steps = 0

  def train_step(self, payload: Any, accumulate_gradients: bool = False, apply_optimizer: bool = True,
                 **kwargs: Any) -> datatypes.Response:
    self.batches.append(payload)
    if apply_optimizer:
      self.optimizer_steps += 1
    return datatypes.Response(metadata={"loss": 1.0 / (1 + self.optimizer_steps), "train_steps": self.optimizer_steps,
                                        "worker_id": self.worker_id})


def shorter_is_better(item: Any) -> float:
  return 1.0 / len(item.completion_tokens)


def main(num_steps: int = 2, group_size: int = 2) -> Dict[str, Any]:
  orch = orchestrator_lib.ClusterOrchestrator()
  rollouts = [SimulatedRolloutWorker("rollout_0"), SimulatedRolloutWorker("rollout_1")]
  trainer = SimulatedTrainerWorker("actor_0")
  for worker in (*rollouts, trainer):
    orch.register_worker(worker)
  print(f"workers: {[(i.worker_id, sorted(i.roles)) for i in orch.worker_infos()]}")
  algo = algorithm_adapter.GRPOAdapter(group_size=group_size, mini_batch_size=2, max_packed_len=32, beta_kl=0.0)
  dataset = [{"prompt_id": f"p{i}", "prompt": text} for i, text in
             enumerate(["Solve 2 + 2", "Solve 3 * 4", "Solve 10 / 2", "Solve 7 - 5"])]
  try:
    program = orch.run(algo=algo, dataset=dataset, reward_fns=[shorter_is_better],
                       assembler=batch_assembly.SequencePackedBatchAssembler(32), num_steps=num_steps)
  finally:
    orch.shutdown()
  print(f"{'step':>4}  {'rollouts':>8}  {'microbatches':>12}  {'reward mean':>11}  {'reward std':>10}")
  for record in program.history:
    print(f"{record.step:>4}  {record.num_rollouts:>8}  {record.num_microbatches:>12}  {record.reward_mean:>11.3f}  "
          f"{record.reward_std:>10.3f}")
  by_worker = {w.worker_id: len(w.served) for w in rollouts}
  print(f"requests served per rollout worker: {by_worker}; trainer saw {len(trainer.batches)} batches, "
        f"{trainer.optimizer_steps} optimizer steps")
  return {"history": program.history, "served": {w.worker_id: list(w.served) for w in rollouts},
          "trainer_batches": len(trainer.batches), "optimizer_steps": trainer.optimizer_steps,
          "states": {w.worker_id: w.state for w in (*rollouts, trainer)}}


if __name__ == "__main__":
  main()
