"""Rollout node of the distributed GSM8K GRPO example
(tunix/experimental/examples/math_gsm8k_dist/run_rollout_node.py).

Hosts a copy of the policy behind the paged generation engine (`NativeSamplerAdapter`; `--engine vllm` uses the
installed vLLM in process instead), wrapped in a `RolloutManager` and a `RolloutWorker`. It is a DESTINATION of
weight transfers: staged buffers behind a host-staged endpoint receive the trainer's parameters and are published
into the serving model between two batches. With `--agentic` every request runs as a one-step episode of the
registered GSM8K environment and agent instead of a plain completion.

  python -m tunix_b200.experimental.examples.math_gsm8k_dist.run_rollout_node \\
      --model tiny --port 50072 --discovery_addrs=control:50070 --max_seq_len 512
"""
from __future__ import annotations

import argparse
import sys

from . import gsm8k, models, node_common


def build_worker(args: argparse.Namespace):
  from tunix_b200.rollout import EngineConfig
  from ...orchestrator import host_staged_handler
  from ...rl.agentic import registry
  from ...rollout import manager as manager_lib
  from ...worker import rollout_worker
  model = models.build_model(args.model, args.seed, args.weights)
  tokenizer = models.build_tokenizer(args.model, args.tokenizer)
  endpoint = host_staged_handler.HostStagedEndpoint()
  worker_id = args.worker_id or "rollout-0"
  if args.engine == "vllm":
    from ...rollout import inprocess_vllm_sampler_adapter as vllm_adapter
    sampler = vllm_adapter.InprocessVllmSamplerAdapter(model, tokenizer, handler=endpoint, worker_id=worker_id)
  else:
    from ...rollout import native_sampler_adapter
    sampler = native_sampler_adapter.NativeSamplerAdapter(
        model, tokenizer, handler=endpoint, worker_id=worker_id,
        engine_config=EngineConfig(page_size=args.page_size, max_batch=args.max_batch, max_seq_len=args.max_seq_len))

  def env_for(request, env_config):
    if not (args.agentic and env_config):
      return None
    env_cls = registry.ENV_REGISTRY.get(env_config.get("env_type", gsm8k.GSM8K_ENV_NAME))
    wanted = ("prompt", "gold_answer", "group_id", "pair_index", "policy_version")
    return env_cls(**{k: env_config[k] for k in wanted if k in env_config})

  def make_manager():
    agent_factory = registry.AGENT_REGISTRY.get(gsm8k.GSM8K_AGENT_NAME) if args.agentic else None
    return manager_lib.RolloutManager(sampler=sampler, tokenizer=tokenizer, chat_parser=None, env_factory=env_for,
                                      agent_factory=agent_factory, max_concurrency=args.max_batch)
  return rollout_worker.RolloutWorker(make_manager, worker_id=worker_id), endpoint, sampler


def main(ctx, argv) -> None:
  parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
  node_common.common_flags(parser, default_port=50072)
  parser.add_argument("--engine", choices=("native", "vllm"), default="native")
  parser.add_argument("--agentic", action="store_true")
  parser.add_argument("--page_size", type=int, default=16)
  parser.add_argument("--max_batch", type=int, default=64)
  parser.add_argument("--max_seq_len", type=int, default=1024)
  args = parser.parse_args(argv)
  worker, endpoint, sampler = build_worker(args)
  node_common.serve_and_wait(ctx, worker, args, "rollout", endpoint, sampler.work_unit)


if __name__ == "__main__":
  node_common.run_standalone(f"{__spec__.name}.main" if __spec__ else "run_rollout_node.main", sys.argv[1:])
