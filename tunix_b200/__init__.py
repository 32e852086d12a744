"""tunix_b200: post-training (SFT / PEFT, DPO / ORPO, distillation, GRPO / PPO, agentic RL) on NVIDIA B200.

The public names mirror the reference's top-level package (tunix/__init__.py:28-67) so that
`from tunix_b200 import PeftTrainer, RLCluster, GRPOLearner` works like `from tunix import ...`.
They are resolved on first access (PEP 562): importing the package itself loads neither torch
nor the CUDA library, which keeps command-line tools and the build check fast.
"""
from __future__ import annotations

import importlib
from typing import Dict, Tuple

__version__ = "0.2.0"

# public name -> (submodule, attribute)
_EXPORTS: Dict[str, Tuple[str, str]] = {
    "CacheConfig": ("common.configs", "CacheConfig"),
    "ClusterConfig": ("common.configs", "ClusterConfig"),
    "RLTrainingConfig": ("common.configs", "RLTrainingConfig"),
    "RolloutConfig": ("common.configs", "RolloutConfig"),
    "TrainingConfig": ("common.configs", "TrainingConfig"),
    "Role": ("common.datatypes", "Role"),
    "DistillationTrainer": ("distillation.distillation_trainer", "DistillationTrainer"),
    "DistillationTrainingConfig": ("distillation.distillation_trainer", "TrainingConfig"),
    "Sampler": ("generate.sampler", "Sampler"),
    "Tokenizer": ("generate.tokenizer_adapter", "Tokenizer"),
    "TokenizerAdapter": ("generate.tokenizer_adapter", "TokenizerAdapter"),
    "PerfMetricsExport": ("perf.export", "PerfMetricsExport"),
    "PerfMetricsConfig": ("perf.metrics", "PerfMetricsConfig"),
    "PerfSpanQuery": ("perf.metrics", "PerfSpanQuery"),
    "AgenticGRPOConfig": ("rl.agentic.agentic_grpo_learner", "GRPOConfig"),
    "AgenticGRPOLearner": ("rl.agentic.agentic_grpo_learner", "GRPOLearner"),
    "GRPOConfig": ("rl.grpo.grpo_learner", "GRPOConfig"),
    "GrpoConfig": ("rl.grpo.grpo_learner", "GrpoConfig"),
    "GRPOLearner": ("rl.grpo.grpo_learner", "GRPOLearner"),
    "GrpoLearner": ("rl.grpo.grpo_learner", "GrpoLearner"),
    "RewardFn": ("rl.grpo.grpo_learner", "RewardFn"),
    "PPOConfig": ("rl.ppo.ppo_learner", "PPOConfig"),
    "PpoConfig": ("rl.ppo.ppo_learner", "PpoConfig"),
    "PPOLearner": ("rl.ppo.ppo_learner", "PPOLearner"),
    "PpoLearner": ("rl.ppo.ppo_learner", "PpoLearner"),
    "MetricsBuffer": ("rl.rl_cluster", "MetricsBuffer"),
    "RLCluster": ("rl.rl_cluster", "RLCluster"),
    "RLEngine": ("rl.rl_cluster", "RLEngine"),
    "CheckpointManager": ("sft.checkpoint_manager", "CheckpointManager"),
    "DPOTrainer": ("sft.dpo.dpo_trainer", "DPOTrainer"),
    "DpoTrainer": ("sft.dpo.dpo_trainer", "DpoTrainer"),
    "DPOTrainingConfig": ("sft.dpo.dpo_trainer", "DPOTrainingConfig"),
    "DpoTrainingConfig": ("sft.dpo.dpo_trainer", "DpoTrainingConfig"),
    "ORPOTrainer": ("sft.dpo.dpo_trainer", "ORPOTrainer"),
    "OrpoTrainer": ("sft.dpo.dpo_trainer", "OrpoTrainer"),
    "ORPOTrainingConfig": ("sft.dpo.dpo_trainer", "ORPOTrainingConfig"),
    "OrpoTrainingConfig": ("sft.dpo.dpo_trainer", "OrpoTrainingConfig"),
    "MetricsLogger": ("sft.metrics_logger", "MetricsLogger"),
    "MetricsLoggerOptions": ("sft.metrics_logger", "MetricsLoggerOptions"),
    "PeftTrainer": ("sft.peft_trainer", "PeftTrainer"),
    # names this framework adds on top of the reference's surface
    "PagedEngine": ("rollout.engine", "PagedEngine"),
    "FlatParamStore": ("dist.fsdp", "FlatParamStore"),
    "AutoModel": ("models.automodel", "AutoModel"),
}

__all__ = sorted(_EXPORTS) + ["__version__"]


def __getattr__(name: str):
  try:
    module, attr = _EXPORTS[name]
  except KeyError:
    raise AttributeError(f"module 'tunix_b200' has no attribute {name!r}") from None
  value = getattr(importlib.import_module(f"{__name__}.{module}"), attr)
  globals()[name] = value      # later lookups skip this hook
  return value


def __dir__():
  return sorted(list(globals()) + list(_EXPORTS))
