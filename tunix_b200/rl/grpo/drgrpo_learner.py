"""Dr. GRPO (https://arxiv.org/abs/2503.20783): advantages `r - mean_g` without the standard
deviation, loss aggregated as `sequence-mean-token-scale` (tunix/rl/grpo/drgrpo_learner.py:28-39)."""
from __future__ import annotations

import dataclasses

from . import grpo_learner as grpo_lib


@dataclasses.dataclass(kw_only=True)
class DrGRPOConfig(grpo_lib.GRPOConfig):
  algo_variant: str = dataclasses.field(default="drgrpo", init=False)
  advantage_estimator: str = dataclasses.field(default="drgrpo", init=False)
  loss_agg_mode: str = "sequence-mean-token-scale"


class DrGRPOLearner(grpo_lib.GRPOLearner):
  """Dr. GRPO learner."""
