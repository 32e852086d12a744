"""A group of rollout engine replicas behind one `BaseRollout` face, with a pluggable traffic
router (tunix/rl/rollout/rollout_engine_group.py:26-90 is a stub; this one round-robins)."""
from __future__ import annotations

from typing import Any, List, Optional

from . import base_rollout
from .rollout_traffic_router import RolloutTrafficRouter


class RolloutEngineGroup(base_rollout.BaseRollout):

  def __init__(self, engines: List[base_rollout.BaseRollout], router: Optional[RolloutTrafficRouter] = None):
    if not engines:
      raise ValueError("RolloutEngineGroup needs at least one engine")
    self.engines = list(engines)
    self.router = router or RolloutTrafficRouter(len(engines))

  def generate(self, prompts, rollout_config, **kwargs):
    return self.engines[self.router.route(prompts)].generate(prompts, rollout_config, **kwargs)

  def get_per_token_logps(self, prompt_tokens, completion_tokens):
    return self.engines[0].get_per_token_logps(prompt_tokens, completion_tokens)

  def update_params(self, params, filter_types=None) -> None:
    for e in self.engines:
      e.update_params(params, filter_types)

  def pad_id(self) -> int:
    return self.engines[0].pad_id()

  def eos_id(self) -> int:
    return self.engines[0].eos_id()

  def model(self) -> Any:
    return self.engines[0].model()
