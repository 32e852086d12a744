"""Shared pytest configuration: the `gpu` marker and helpers for building the kernel library."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (run with `-m gpu` on a B200)")


def pytest_collection_modifyitems(config, items):
  import torch
  if torch.cuda.is_available():
    return
  skip = pytest.mark.skip(reason="no CUDA device")
  for item in items:
    if "gpu" in item.keywords:
      item.add_marker(skip)


@pytest.fixture(scope="session")
def kernel_lib():
  """Builds (if needed) and loads the sm_100a kernel library; fails loudly when impossible."""
  from tunix_b200 import build_kernels
  from tunix_b200.ops import _lib
  if not _lib.lib_path().exists():
    build_kernels.build()
  return _lib.require()
