"""GRPO entry point (tunix/cli/grpo_main.py:43-199).

`training_mode: "grpo"` (default) runs single-turn GRPO; `"agentic_grpo"` runs the asynchronous
multi-turn learner and also reads `agentic_grpo_config` (GRPOConfig fields plus `max_turns`,
`per_turn_timeout_secs`), `chat_parser_class`, `agent_class` / `env_class` (dotted paths) with
`agent_kwargs` / `env_kwargs`.

  python -m tunix_b200.cli.grpo_main base_config.yaml model_config.model_source=dummy data_source=synthetic ...
"""
from __future__ import annotations

import dataclasses
import logging
import sys
from typing import Any, Dict

from . import base_rl_pipeline


class GrpoPipeline(base_rl_pipeline.BasePipeline):
  def _default_training_mode(self) -> str:
    return "grpo"

  def _create_agentic_grpo_config(self):
    from ..rl.agentic.agentic_grpo_learner import GRPOConfig
    cfg = dict(self.config.get("agentic_grpo_config") or {})
    if "episode_timeout" not in cfg:
      per_turn = cfg.pop("per_turn_timeout_secs", None)
      if per_turn is not None:
        cfg["episode_timeout"] = per_turn * cfg.get("max_turns", 1)
    cfg.setdefault("max_response_length", (self.config.get("rollout_config") or {}).get("total_generation_steps", 8192))
    cfg.pop("max_turns", None)
    valid = {f.name for f in dataclasses.fields(GRPOConfig)}
    return GRPOConfig(**{k: v for k, v in cfg.items() if k in valid})

  def _run(self, mode: str = "grpo"):
    tokenizer = self._get_tokenizer()
    chat_parser = self._create_chat_parser(tokenizer)
    dataset, _ = self._get_dataset(tokenizer)
    rl_engine = self.create_rl_engine(tokenizer)
    if mode == "grpo":
      from ..rl.grpo import grpo_learner
      learner = grpo_learner.GRPOLearner(rl_engine=rl_engine, reward_fns=self.obtain_reward_fn(),
                                         algo_config=grpo_learner.GRPOConfig(**(self.config.get("grpo_config") or {})))
      learner.train(dataset)
      return learner
    if mode != "agentic_grpo":
      raise ValueError(f"Unsupported training_mode {mode!r}")
    from ..rl.agentic.agentic_grpo_learner import GRPOLearner
    kw: Dict[str, Any] = dict(rl_engine=rl_engine, algo_config=self._create_agentic_grpo_config(),
                              reward_fns=self.obtain_reward_fn() if self.config.get("reward_functions") else None,
                              chat_parser=chat_parser)
    if self.config.get("agent_class"):
      kw["agent_class"] = self._load_class_from_path(self.config["agent_class"])
      kw["agent_kwargs"] = dict(self.config.get("agent_kwargs") or {})
    if self.config.get("env_class"):
      kw["env_class"] = self._load_class_from_path(self.config["env_class"])
      kw["env_kwargs"] = dict(self.config.get("env_kwargs") or {})
    learner = GRPOLearner(**kw)
    learner.train(dataset)
    return learner


def main(argv, **kwargs):
  pipeline = GrpoPipeline(argv, **kwargs)
  logging.info("--- Launching GRPO pipeline with following config ---\n%r\n--------------------------", pipeline.config)
  return pipeline.run_trainer()


if __name__ == "__main__":
  logging.basicConfig(level=logging.INFO)
  main(sys.argv)
