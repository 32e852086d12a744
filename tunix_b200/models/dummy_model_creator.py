"""Random-weight model of a given config (role of tunix/models/dummy_model_creator.py:30-92):
every parameter ~ N(0, scale) drawn on the target device from a seeded generator, norm scales
at their identity value; used by tests, benchmarks and the CLI's `model_source: dummy`."""
from __future__ import annotations

from typing import Callable, Optional

import torch


def create_dummy_model(model_class: Callable, config, mesh=None, dtype: Optional[torch.dtype] = None,
                       random_seed: int = 0, scale: float = 0.02, device: Optional[str] = None):
  del mesh   # sharding is applied afterwards by dist.fsdp.shard_model
  device = device or ("cuda" if torch.cuda.is_available() else "cpu")
  with torch.device(device):
    model = model_class(config)
  if dtype is not None:
    model = model.to(dtype)
  model.init_weights(seed=random_seed, scale=scale)
  return model
