"""Reward value plus diagnostic metadata (tunix/rl/agentic/rewards/reward_types.py:24-65)."""
from __future__ import annotations

import dataclasses
from typing import Any, Dict


@dataclasses.dataclass
class RewardOutput:
  reward: float
  metadata: Dict[str, Any] = dataclasses.field(default_factory=dict)
