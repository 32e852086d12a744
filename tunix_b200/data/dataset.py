"""Small random-access dataset with lazy transforms (the part of the `grain` MapDataset /
IterDataset surface that the reference's CLI and example pipelines rely on:
tunix/cli/utils/data.py:168-261, tunix/examples/data/*.py)."""
from __future__ import annotations

import random
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence

import numpy as np


def default_batch_fn(items: Sequence[Any]) -> Any:
  """Dicts are batched per key: arrays / numbers are stacked, everything else becomes a list."""
  first = items[0]
  if isinstance(first, dict):
    out: Dict[str, Any] = {}
    for k in first:
      vals = [it[k] for it in items]
      v0 = vals[0]
      if isinstance(v0, np.ndarray) and all(isinstance(v, np.ndarray) and v.shape == v0.shape for v in vals):
        out[k] = np.stack(vals)
      elif isinstance(v0, (int, float, np.number)) and not isinstance(v0, bool):
        out[k] = np.asarray(vals)
      else:
        out[k] = list(vals)
    return out
  if isinstance(first, np.ndarray):
    return np.stack(items)
  return list(items)


class ListDataset:
  """Random-access dataset; transforms return new datasets and run at access time."""

  def __init__(self, source: Sequence[Any], _index: Optional[Sequence[int]] = None,
               _fns: Optional[List[Callable[[Any], Any]]] = None):
    self._source = source
    self._index = list(range(len(source))) if _index is None else list(_index)
    self._fns = list(_fns or [])

  def __len__(self) -> int:
    return len(self._index)

  def _get(self, i: int) -> Any:
    x = self._source[self._index[i]]
    for f in self._fns:
      x = f(x)
    return x

  def __getitem__(self, i):
    if isinstance(i, slice):
      return ListDataset(self._source, self._index[i], self._fns)
    if i < 0:
      i += len(self)
    if not 0 <= i < len(self):
      raise IndexError(i)
    return self._get(i)

  def __iter__(self) -> Iterator[Any]:
    return (self._get(i) for i in range(len(self)))

  def map(self, fn: Callable[[Any], Any]) -> "ListDataset":
    return ListDataset(self._source, self._index, self._fns + [fn])

  def filter(self, pred: Callable[[Any], bool]) -> "ListDataset":
    keep = [self._index[i] for i in range(len(self)) if pred(self._get(i))]
    return ListDataset(self._source, keep, self._fns)

  def shuffle(self, seed: int = 0) -> "ListDataset":
    idx = list(self._index)
    random.Random(seed).shuffle(idx)
    return ListDataset(self._source, idx, self._fns)

  def repeat(self, num_epochs: Optional[int] = 1) -> "ListDataset":
    if num_epochs is None:
      raise ValueError("infinite repeat needs to_iter_dataset().repeat()")
    return ListDataset(self._source, self._index * int(num_epochs), self._fns)

  def to_iter_dataset(self) -> "IterDataset":
    return IterDataset(lambda: iter(self))

  def batch(self, batch_size: int, drop_remainder: bool = False, batch_fn: Optional[Callable] = None) -> "IterDataset":
    return self.to_iter_dataset().batch(batch_size, drop_remainder=drop_remainder, batch_fn=batch_fn)


class IterDataset:
  """Re-iterable stream (each `iter()` restarts from the beginning)."""

  def __init__(self, make_iter: Callable[[], Iterator[Any]]):
    self._make = make_iter

  def __iter__(self) -> Iterator[Any]:
    return self._make()

  def map(self, fn: Callable[[Any], Any]) -> "IterDataset":
    return IterDataset(lambda: (fn(x) for x in self._make()))

  def filter(self, pred: Callable[[Any], bool]) -> "IterDataset":
    return IterDataset(lambda: (x for x in self._make() if pred(x)))

  def batch(self, batch_size: int, drop_remainder: bool = False, batch_fn: Optional[Callable] = None) -> "IterDataset":
    fn = batch_fn or default_batch_fn

    def gen():
      buf = []
      for x in self._make():
        buf.append(x)
        if len(buf) == batch_size:
          yield fn(buf)
          buf = []
      if buf and not drop_remainder:
        yield fn(buf)
    return IterDataset(gen)

  def take(self, n: int) -> "IterDataset":
    def gen():
      for i, x in enumerate(self._make()):
        if i >= n:
          return
        yield x
    return IterDataset(gen)
