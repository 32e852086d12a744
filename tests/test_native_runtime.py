"""Native host runtime (packer, parallel reads, asynchronous writer) against the Python equivalents."""
import os

import numpy as np
import pytest
import torch

from tunix_b200.runtime import native


def test_ffd_pack_matches_python_and_respects_limits():
  rng = np.random.default_rng(0)
  for trial in range(20):
    n = int(rng.integers(1, 200))
    lengths = rng.integers(1, 900, size=n).tolist()
    pack, budget, segs = int(rng.integers(1, 9)), int(rng.integers(500, 3000)), int(rng.integers(1, 12))
    want = native.ffd_pack_py(lengths, pack, budget, segs)
    got = native.ffd_pack(lengths, pack, budget, segs)
    assert got == want, trial
    loads, counts = [0] * pack, [0] * pack
    for i, b in enumerate(got):
      if b >= 0:
        loads[b] += lengths[i]
        counts[b] += 1
    assert max(loads) <= budget and max(counts) <= segs
  assert native.ffd_pack([], 2, 10, 2) == []
  assert native.ffd_pack([50, 50], 1, 10, 4) == [-1, -1]


def test_packer_is_used_by_the_rl_sequence_packer():
  from tunix_b200.rl import utils as rl_utils
  items = [{"prompt_ids": [1] * p, "completion_ids": [2] * c} for p, c in [(5, 9), (3, 3), (8, 8), (2, 1), (7, 2)]]
  bins, left = rl_utils._fill_one_chunk(items, pack_size=2, budget=20, max_segments=3)
  assert sum(len(b) for b in bins) + len(left) == len(items)
  for b in bins:
    assert sum(len(i["prompt_ids"]) + len(i["completion_ids"]) for i in b) <= 20


def test_parallel_read_and_async_writer(tmp_path):
  rng = np.random.default_rng(1)
  blob = rng.integers(0, 255, size=(3 << 20) + 123, dtype=np.uint8)
  path = str(tmp_path / "blob.bin")
  blob.tofile(path)
  dst = torch.empty(1 << 20, dtype=torch.uint8)
  native.read_into(path, 1000, dst.numel(), dst.data_ptr(), threads=4)
  assert np.array_equal(dst.numpy(), blob[1000:1000 + (1 << 20)])
  with pytest.raises(OSError):
    native.read_into(path, blob.nbytes - 10, 1000, dst.data_ptr())       # past the end of the file
  with pytest.raises(OSError):
    native.read_into(str(tmp_path / "missing"), 0, 10, dst.data_ptr())

  w = native.AsyncWriter(threads=3)
  parts = {f"part{i}.bin": torch.from_numpy(rng.integers(0, 255, size=50000 + i, dtype=np.uint8)) for i in range(8)}
  for name, t in parts.items():
    w.submit(str(tmp_path / name), t)
  w.submit(str(tmp_path / "small.txt"), b"hello")
  w.wait()
  for name, t in parts.items():
    assert np.array_equal(np.fromfile(tmp_path / name, dtype=np.uint8), t.numpy())
  assert (tmp_path / "small.txt").read_bytes() == b"hello"
  assert not [f for f in os.listdir(tmp_path) if ".tmp." in f]
  w.submit(str(tmp_path / "no_such_dir" / "x.bin"), b"data")
  with pytest.raises(OSError):
    w.wait()
  w.submit(str(tmp_path / "after_error.bin"), b"ok")       # the writer keeps working after a failure
  w.wait()
  assert (tmp_path / "after_error.bin").read_bytes() == b"ok"
  w.close()
