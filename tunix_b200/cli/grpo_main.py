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

  def _pluggable(self, kind: str) -> Dict[str, Any]:
    """`{kind}_class` (a dotted path) and `{kind}_kwargs` of the config as learner keyword arguments."""
    path = self.config.get(f"{kind}_class")
    if not path:
      return {}
    return {f"{kind}_class": self._load_class_from_path(path), f"{kind}_kwargs": dict(self.config.get(f"{kind}_kwargs") or {})}

  def _single_turn_learner(self, rl_engine, chat_parser):
    from ..rl.grpo import grpo_learner
    algo = grpo_learner.GRPOConfig(**(self.config.get("grpo_config") or {}))
    return grpo_learner.GRPOLearner(rl_engine=rl_engine, reward_fns=self.obtain_reward_fn(), algo_config=algo)

  def _agentic_learner(self, rl_engine, chat_parser):
    from ..rl.agentic import agentic_grpo_learner
    rewards = self.obtain_reward_fn() if self.config.get("reward_functions") else None
    return agentic_grpo_learner.GRPOLearner(rl_engine=rl_engine, algo_config=self._create_agentic_grpo_config(),
                                            reward_fns=rewards, chat_parser=chat_parser, **self._pluggable("agent"),
                                            **self._pluggable("env"))

  _LEARNERS = {"grpo": "_single_turn_learner", "agentic_grpo": "_agentic_learner"}

  def _run(self, mode: str = "grpo"):
    if mode not in self._LEARNERS:
      raise ValueError(f"Unsupported training_mode {mode!r}")
    tokenizer = self._get_tokenizer()
    chat_parser = self._create_chat_parser(tokenizer)
    dataset, _ = self._get_dataset(tokenizer)
    learner = getattr(self, self._LEARNERS[mode])(self.create_rl_engine(tokenizer), chat_parser)
    learner.train(dataset)
    return learner


def main(argv, **kwargs):
  pipeline = GrpoPipeline(argv, **kwargs)
  logging.info("--- Launching GRPO pipeline with following config ---\n%r\n--------------------------", pipeline.config)
  return pipeline.run_trainer()


if __name__ == "__main__":
  logging.basicConfig(level=logging.INFO)
  main(sys.argv)
