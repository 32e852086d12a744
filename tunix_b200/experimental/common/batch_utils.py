"""Running a function over a batch in bounded pieces (tunix/experimental/common/batch_utils.py)."""
from __future__ import annotations

from typing import Any, Callable, Optional

import numpy as np


def apply_chunked(fn: Callable[..., Any], chunk_size: Optional[int], *input_arrays: np.ndarray) -> np.ndarray:
  """`fn(*arrays)` evaluated on row ranges of at most `chunk_size` rows (axis 0 of every array), results
  concatenated - identical to one call when `fn` treats rows independently, with peak memory bounded by
  the chunk. `chunk_size=None` or a chunk that covers the batch is a single call."""
  if not input_arrays:
    raise ValueError("apply_chunked needs at least one array")
  rows = {int(a.shape[0]) if getattr(a, "ndim", 0) >= 1 else None for a in input_arrays}
  if None in rows:
    raise ValueError("every input must have a batch dimension")
  if len(rows) != 1:
    raise ValueError(f"inputs disagree on the batch size: {sorted(rows)}")
  if chunk_size is not None and chunk_size <= 0:
    raise ValueError(f"chunk_size must be positive, got {chunk_size}")
  n = rows.pop()
  if not chunk_size or chunk_size >= n:
    return np.asarray(fn(*input_arrays))
  return np.concatenate([np.asarray(fn(*(a[lo:lo + chunk_size] for a in input_arrays)))
                         for lo in range(0, n, chunk_size)], axis=0)
