"""Process-environment probes (the role of tunix/utils/env_utils.py).

The reference asks "is this the internal build / a Pathways controller?". On this platform the
questions are about the launcher and the device: were we started by torchrun, is a B200 visible,
is the compiled kernel library there, are peer mappings between the local GPUs allowed.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

TP_AXIS_NAME = os.environ.get("TUNIX_TP_AXIS_NAME", "tp")
SGLANG_JAX_TP_AXIS_NAME = os.environ.get("SGLANG_JAX_TP_AXIS_NAME", "tensor")   # config surface kept for recipes


def launched_by_torchrun() -> bool:
  return all(k in os.environ for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))


def rank_info() -> Dict[str, int]:
  return {"rank": int(os.environ.get("RANK", "0")), "world_size": int(os.environ.get("WORLD_SIZE", "1")),
          "local_rank": int(os.environ.get("LOCAL_RANK", "0"))}


def setup_sharding_environment() -> None:
  """Start-up settings every rank needs before the first allocation: the rendezvous address defaults to
  loopback (single node), and the caching allocator grows segments in place so that the large flat
  parameter / gradient buffers do not fragment it."""
  os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
  os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


def is_internal_env() -> bool:
  return False


def is_pathways_initialized() -> bool:
  """There is no single-controller runtime here: every GPU has its own process."""
  return False


def gpu_name(index: Optional[int] = None) -> Optional[str]:
  import torch
  if not torch.cuda.is_available():
    return None
  return torch.cuda.get_device_name(torch.cuda.current_device() if index is None else index)


def is_blackwell() -> bool:
  import torch
  return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] >= 10


def kernels_built() -> bool:
  from ..ops import _lib
  return _lib.lib_path().exists()


def peer_access_matrix():
  """[n, n] booleans: can GPU i map GPU j's memory (NVLink / NVSwitch peer access)."""
  import torch
  n = torch.cuda.device_count() if torch.cuda.is_available() else 0
  return [[i == j or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]
