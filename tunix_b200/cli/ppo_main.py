"""PPO entry point (tunix/cli/ppo_main.py:35-120): actor + critic (score head on a second
backbone, `critic_model_config` required) with reward functions or a reward model.

  python -m tunix_b200.cli.ppo_main base_config.yaml critic_model_config='{...}' ...
"""
from __future__ import annotations

import logging
import sys

from . import base_rl_pipeline


class PpoPipeline(base_rl_pipeline.BasePipeline):
  def _default_training_mode(self) -> str:
    return "ppo"

  def _run(self, mode: str = "ppo"):
    if mode != "ppo":
      raise ValueError(f"Unsupported training_mode {mode!r}")
    if not self.config.get("critic_model_config"):
      raise ValueError("PPO needs critic_model_config")
    if not (self.config["rl_training_config"] or {}).get("critic_optimizer_config"):
      raise ValueError("PPO needs rl_training_config.critic_optimizer_config")
    from ..rl.ppo import ppo_learner
    tokenizer = self._get_tokenizer()
    dataset, _ = self._get_dataset(tokenizer)
    rl_engine = self.create_rl_engine(tokenizer)
    learner = ppo_learner.PPOLearner(rl_engine=rl_engine, reward_fns=self.obtain_reward_fn(),
                                     algo_config=ppo_learner.PPOConfig(**(self.config.get("ppo_config") or {})))
    learner.train(dataset)
    return learner


def main(argv, **kwargs):
  pipeline = PpoPipeline(argv, **kwargs)
  logging.info("--- Launching PPO pipeline with following config ---\n%r\n--------------------------", pipeline.config)
  return pipeline.run_trainer()


if __name__ == "__main__":
  logging.basicConfig(level=logging.INFO)
  main(sys.argv)
