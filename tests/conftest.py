"""Shared pytest configuration: the `gpu` marker and helpers for building the kernel library."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
  config.addinivalue_line("markers", "gpu: needs a CUDA device (run with `-m gpu` on a B200)")


_DEFAULT_TEST_TIMEOUT_S = 900      # multi-rank tests bound their child processes at 600 s themselves


def pytest_collection_modifyitems(config, items):
  # no test may hang the suite: where the pytest-timeout plugin is installed every test without a limit of its
  # own gets one (a stuck event loop or a lost collective then fails that test instead of the whole run)
  if config.pluginmanager.hasplugin("timeout"):
    for item in items:
      if item.get_closest_marker("timeout") is None:
        item.add_marker(pytest.mark.timeout(_DEFAULT_TEST_TIMEOUT_S))
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
