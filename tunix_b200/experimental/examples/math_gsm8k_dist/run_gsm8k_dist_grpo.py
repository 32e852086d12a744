"""Control plane of the distributed GSM8K GRPO example
(tunix/experimental/examples/math_gsm8k_dist/run_gsm8k_dist_grpo.py).

This process holds no model. It waits for the worker nodes to announce themselves, turns every announcement into a
remote handle, registers the handles with a `ClusterOrchestrator`, sends the GRPO loss to the trainer node, builds a
`WeightSyncCoordinator` whose host-staged handler knows each node's transfer endpoint, and runs
`StandardRLProgram`: rollouts from the rollout nodes, reference log-probs from the inference node when the KL
coefficient is non-zero, optimizer steps on the trainer node, and a weight-sync round after every step.

One machine, four terminals (or one launcher with four `--process` sections):

  python -m tunix_b200.experimental.examples.math_gsm8k_dist.run_gsm8k_dist_grpo \\
      --discovery_id=control --discovery_port=50070 --steps 4 --num_generations 4
  python -m tunix_b200.experimental.examples.math_gsm8k_dist.run_trainer_node   --discovery_addrs=control:50070 --lr 1e-2
  python -m tunix_b200.experimental.examples.math_gsm8k_dist.run_rollout_node   --discovery_addrs=control:50070
  python -m tunix_b200.experimental.examples.math_gsm8k_dist.run_inference_node --discovery_addrs=control:50070

Across machines the nodes serve on `--host 0.0.0.0` and the discovery ids are host names (or, in a JobSet, job
names with `--process_executor=...K8sExecutor`).
"""
from __future__ import annotations

import argparse
import logging
import sys
import threading
from typing import Any, Callable, Dict, List, Optional

from ...common import datatypes
from ...orchestrator import (algorithm_adapter, batch_assembly, host_staged_handler, orchestrator as orchestrator_lib,
                             rl_program, weight_sync_coordinator)
from ...worker import remote_execution
from . import gsm8k, models, node_common


class RemoteMember:
  """A weight-sync participant that lives behind a handle: every phase the coordinator calls becomes a remote call
  with the same name (the phases are coroutines on both sides)."""

  def __init__(self, worker_id: str, handle: remote_execution.ActorHandle):
    self.worker_id, self._handle = worker_id, handle

  def info(self) -> datatypes.WorkerInfo:
    return datatypes.WorkerInfo(worker_id=self.worker_id, roles=frozenset(), resources={"remote": True})

  def __getattr__(self, name: str) -> Callable[..., Any]:
    if name.startswith("_"):
      raise AttributeError(name)

    async def remote_phase(*args: Any, **kwargs: Any) -> Any:
      return await self._handle.asubmit(name, *args, **kwargs)
    remote_phase.__name__ = name
    return remote_phase


class Cluster:
  """Announcements collected from discovery until the expected set of nodes is there."""

  def __init__(self, resolve_host: Callable[[str], str] = lambda host: "127.0.0.1"):
    self._resolve = resolve_host
    self._cv = threading.Condition()
    self.nodes: List[Dict[str, Any]] = []

  def accept(self, hostname: str, discovery_port: int, metadata: bytes) -> None:
    info = node_common.parse_announcement(metadata)
    info["host"] = self._resolve(hostname)
    info["handle"] = remote_execution.ActorHandle.from_address(f"grpc://{info['host']}:{info['rpc_port']}")
    logging.info("discovered %s node %s at %s:%d", info["role"], info["worker_id"], info["host"], info["rpc_port"])
    with self._cv:
      self.nodes.append(info)
      self._cv.notify_all()

  def by_role(self, role: str) -> List[Dict[str, Any]]:
    return [n for n in self.nodes if n["role"] == role]

  def wait(self, rollouts: int, need_reference: bool, timeout_s: float) -> None:
    def complete() -> bool:
      return (len(self.by_role("actor")) >= 1 and len(self.by_role("rollout")) >= rollouts
              and (not need_reference or len(self.by_role("reference")) >= 1))
    with self._cv:
      if not self._cv.wait_for(complete, timeout_s):
        have = {r: len(self.by_role(r)) for r in ("actor", "rollout", "reference")}
        raise SystemExit(f"after {timeout_s:.0f} s the cluster is incomplete: {have}")


def grpo_loss(algo_config: Any, pad_id: int, eos_id: int) -> Callable[..., Any]:
  """The loss the trainer node will run; it travels there by value, the registry lookup happens on the node."""
  def loss(model, train_example):
    from tunix_b200.rl import function_registry
    fn = function_registry.get_policy_loss_fn("grpo")
    return fn(model, train_example.to_tensors(), algo_config=algo_config, pad_id=pad_id, eos_id=eos_id)
  return loss


def decoded_reward(reward: Callable[[Any], float], tokenizer: Any) -> Callable[[Any], float]:
  def score(item: Any) -> float:
    item.metadata["completion_text"] = tokenizer.decode([int(t) for t in item.completion_tokens])
    return float(reward(item))
  return score


def build_coordinator(cluster: Cluster, timeout_s: float) -> weight_sync_coordinator.WeightSyncCoordinator:
  handler = host_staged_handler.HostStagedHandler(timeout_s=timeout_s)
  ends = cluster.by_role("actor") + cluster.by_role("rollout")
  for node in ends:
    handler.register_endpoint(node["unit"], (node["host"], node["staged_port"]))
  member = lambda n: RemoteMember(n["worker_id"], n["handle"])                       # noqa: E731
  return weight_sync_coordinator.WeightSyncCoordinator(
      handler, sources=[member(n) for n in cluster.by_role("actor")],
      destinations=[member(n) for n in cluster.by_role("rollout")])


def run(ctx: Any, args: argparse.Namespace) -> List[Any]:
  from tunix_b200.rl.grpo.grpo_learner import GRPOConfig
  need_reference = args.beta != 0.0
  cluster = Cluster()
  ctx.ipc.discovery.on_register(cluster.accept)
  cluster.wait(args.rollout_nodes, need_reference, args.wait_s)
  tokenizer = models.build_tokenizer(args.model, args.tokenizer)
  pad, eos = models.pad_and_eos(tokenizer)

  orch = orchestrator_lib.ClusterOrchestrator(weight_sync_coordinator=build_coordinator(cluster, args.transfer_timeout_s))
  for node in cluster.nodes:
    if node["role"] == "reference" and not need_reference:
      continue
    orch.register_worker_handle(node["worker_id"], [node["role"]], node["handle"])
  algo_config = GRPOConfig(num_generations=args.num_generations, beta=args.beta, epsilon=args.epsilon)
  trainer = cluster.by_role("actor")[0]["handle"]
  trainer.submit("with_loss_fn", grpo_loss(algo_config, pad, eos), True)
  trainer.submit("with_gen_model_input_fn", lambda example: {"train_example": example})

  algo = algorithm_adapter.GRPOAdapter(group_size=args.num_generations, mini_batch_size=args.mini_batch_size,
                                       clip_epsilon=args.epsilon, beta_kl=args.beta)
  history: List[Any] = []

  def report(step: int, record: Any) -> None:
    history.append(record)
    logging.info("step %d: policy version %s, %s rollouts, mean reward %s", step,
                 getattr(record, "policy_version", "?"), getattr(record, "num_rollouts", "?"),
                 getattr(record, "mean_reward", "?"))
  program = rl_program.StandardRLProgram(
      algo, reward_fns=[decoded_reward(gsm8k.make_reward_fn(args.reward), tokenizer)],
      assembler=batch_assembly.GRPOTrainExampleAssembler(
          batch_size=args.mini_batch_size, max_prompt_length=args.max_prompt_length,
          max_response_length=args.max_response_length, pad_id=pad),
      max_staleness=args.max_staleness, on_step_end=report)
  generation = {"max_generation_steps": args.max_response_length, "temperature": args.temperature}
  tasks = gsm8k.load_tasks(args.data, args.num_prompts, args.seed)
  dataset = gsm8k.prompt_items(tasks, generation, agentic=args.agentic)
  try:
    with orch:
      orch.run_program(program, dataset, num_steps=args.steps)
  finally:
    node_common.stop.set()          # node bodies that share this OS process end with the run
  return program.history or history


def parse_args(argv: List[str]) -> argparse.Namespace:
  p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
  p.add_argument("--model", default="tiny")
  p.add_argument("--tokenizer", default=None)
  p.add_argument("--data", default=None, help="GSM8K-format JSON lines; synthetic word problems when absent")
  p.add_argument("--num_prompts", type=int, default=64)
  p.add_argument("--steps", type=int, default=4)
  p.add_argument("--num_generations", type=int, default=4)
  p.add_argument("--mini_batch_size", type=int, default=4)
  p.add_argument("--beta", type=float, default=0.04)
  p.add_argument("--epsilon", type=float, default=0.2)
  p.add_argument("--temperature", type=float, default=1.0)
  p.add_argument("--reward", choices=("answer", "contains", "length"), default="answer")
  p.add_argument("--agentic", action="store_true")
  p.add_argument("--max_prompt_length", type=int, default=256)
  p.add_argument("--max_response_length", type=int, default=256)
  p.add_argument("--max_staleness", type=int, default=1)
  p.add_argument("--rollout_nodes", type=int, default=1)
  p.add_argument("--wait_s", type=float, default=600.0)
  p.add_argument("--transfer_timeout_s", type=float, default=300.0)
  p.add_argument("--seed", type=int, default=0)
  return p.parse_args(argv)


def main(ctx: Any, argv: List[str]) -> List[Any]:
  return run(ctx, parse_args(argv))


if __name__ == "__main__":
  node_common.run_standalone(f"{__spec__.name}.main" if __spec__ else "run_gsm8k_dist_grpo.main", sys.argv[1:])
