"""Minimal safetensors reader / writer on mmap (no dependency on the `safetensors` package).

File format: 8-byte little-endian header length, JSON header {name: {dtype, shape,
data_offsets}}, then the raw little-endian tensor bytes. The reader maps the file and hands
out zero-copy torch views, so a 16 GB shard costs no host copy before the H2D transfer.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from typing import Dict, Iterator, List, Mapping, Optional, Tuple

import numpy as np
import torch

_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
           "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
           "BOOL": torch.bool, "F8_E4M3": torch.float8_e4m3fn, "F8_E5M2": torch.float8_e5m2}
_NAMES = {v: k for k, v in _DTYPES.items()}


class SafeTensorsFile:
  """One mapped `.safetensors` file."""

  def __init__(self, path: str):
    self.path = path
    self._f = open(path, "rb")
    (n,) = struct.unpack("<Q", self._f.read(8))
    self.header: Dict[str, dict] = json.loads(self._f.read(n))
    self.metadata = self.header.pop("__metadata__", {})
    self._data_start = 8 + n
    self._mm = mmap.mmap(self._f.fileno(), 0, access=mmap.ACCESS_READ)

  def keys(self) -> List[str]:
    return list(self.header)

  def shape(self, name: str) -> Tuple[int, ...]:
    return tuple(self.header[name]["shape"])

  def get(self, name: str) -> torch.Tensor:
    info = self.header[name]
    dt = _DTYPES[info["dtype"]]
    b, e = info["data_offsets"]
    if e == b:
      return torch.empty(info["shape"], dtype=dt)
    buf = memoryview(self._mm)[self._data_start + b:self._data_start + e]
    # torch.frombuffer wants a writable buffer for no warning; a read-only view is fine for copies
    import warnings
    with warnings.catch_warnings():
      warnings.simplefilter("ignore")
      t = torch.frombuffer(buf, dtype=dt)
    return t.view(info["shape"])

  def close(self):
    try:
      self._mm.close()
    except BufferError:      # views still alive; the map goes away with them
      pass
    self._f.close()

  def __enter__(self):
    return self

  def __exit__(self, *a):
    self.close()


def list_files(path: str) -> List[str]:
  """`path` is a file, or a directory with `*.safetensors` (sharded checkpoints use an index)."""
  if os.path.isfile(path):
    return [path]
  idx = os.path.join(path, "model.safetensors.index.json")
  if os.path.exists(idx):
    with open(idx) as f:
      files = sorted(set(json.load(f)["weight_map"].values()))
    return [os.path.join(path, f) for f in files]
  files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
  if not files:
    raise FileNotFoundError(f"no .safetensors files under {path}")
  return [os.path.join(path, f) for f in files]


def iter_tensors(path: str) -> Iterator[Tuple[str, torch.Tensor]]:
  for fp in list_files(path):
    f = SafeTensorsFile(fp)
    for k in f.keys():
      yield k, f.get(k)


def save_file(tensors: Mapping[str, torch.Tensor], path: str, metadata: Optional[Dict[str, str]] = None) -> None:
  header, offset, blobs = {}, 0, []
  if metadata:
    header["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
  for name in sorted(tensors):
    t = tensors[name].detach().cpu().contiguous()
    n = t.numel() * t.element_size()
    header[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape), "data_offsets": [offset, offset + n]}
    blobs.append(t)
    offset += n
  hj = json.dumps(header, separators=(",", ":")).encode()
  hj += b" " * ((8 - len(hj) % 8) % 8)
  tmp = path + ".tmp"
  with open(tmp, "wb") as f:
    f.write(struct.pack("<Q", len(hj)))
    f.write(hj)
    for t in blobs:
      f.write(t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b"")   # reshape: 0-dim scalars too
  os.replace(tmp, path)
