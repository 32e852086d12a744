"""Reading and writing parameter trees in the Orbax on-disk layout.

A checkpointable directory (`<root>/<step>/model_params`, `.../optimizer_state`) holds
`_METADATA` (tree structure keyed by stringified key tuples), `_sharding`,
`array_metadatas/process_<r>` and the arrays. Arrays are written as plain zarr-v2 directories
(`<a.b.c>/.zarray` + chunk files) - the variant Orbax itself produces when OCDBT is disabled
(tunix/sft/checkpoint_manager.py:156-159) and reads back transparently. Reading also accepts
the OCDBT key-value-store variant (`manifest.ocdbt` + `d/*`), see `ocdbt.py`.

Trees are flat dicts `{("layers", 0, "attn", "q_proj", "w", "value"): ndarray}`: string keys are
dict keys (key_type 2), ints are sequence indices (key_type 1).
"""
from __future__ import annotations

import base64
import dataclasses
import ctypes
import ctypes.util
import json
import os
import time
from typing import Any, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple, Union

import numpy as np
import torch

Key = Tuple[Union[str, int], ...]


@dataclasses.dataclass
class ShardedArray:
  """A leaf that is split over the ranks of a job: this process holds `local`, one chunk of a larger
  array of shape `global_shape` cut on a regular grid of `chunk_shape` blocks, at grid position
  `chunk_index`. On disk that is an ordinary zarr array whose chunk files come from different
  processes - the form Orbax writes for an array sharded over hosts - so nothing is gathered to save it.
  """
  local: torch.Tensor
  global_shape: Tuple[int, ...]
  chunk_shape: Tuple[int, ...]
  chunk_index: Tuple[int, ...]

  def detach(self) -> "ShardedArray":
    return self

_ZARR_DTYPES = {
    "float32": "<f4", "float64": "<f8", "float16": "<f2", "bfloat16": "bfloat16", "int32": "<i4", "int64": "<i8",
    "int16": "<i2", "int8": "|i1", "uint8": "|u1", "bool": "|b1", "uint32": "<u4", "uint16": "<u2",
}
_NP_FROM_ZARR = {v: k for k, v in _ZARR_DTYPES.items()}


def key_to_str(key: Key) -> str:
  return "(" + ", ".join(repr(k) for k in key) + ("," if len(key) == 1 else "") + ")"


def param_name(key: Key) -> str:
  return ".".join(str(k) for k in key)


def _tensor_to_bytes(t: torch.Tensor) -> Tuple[bytes, str, List[int]]:
  t = t.detach()
  if t.is_cuda:
    t = t.cpu()
  t = t.contiguous()
  shape = list(t.shape)
  if t.dtype == torch.bfloat16:
    return t.view(torch.int16).numpy().tobytes(), "bfloat16", shape
  a = t.numpy()
  return a.tobytes(), _ZARR_DTYPES[str(a.dtype)], shape


def _bytes_to_tensor(buf: bytes, zdtype: str, shape: Sequence[int]) -> torch.Tensor:
  if zdtype == "bfloat16":
    a = np.frombuffer(buf, dtype=np.int16).reshape(shape).copy()
    return torch.from_numpy(a).view(torch.bfloat16)
  name = _NP_FROM_ZARR.get(zdtype)
  if name is None:
    a = np.frombuffer(buf, dtype=np.dtype(zdtype)).reshape(shape).copy()
  else:
    a = np.frombuffer(buf, dtype=np.dtype(name)).reshape(shape).copy()
  return torch.from_numpy(a)


# ---------------------------------------------------------------------------- zstd (optional)
_zstd = None


def _load_zstd():
  global _zstd
  if _zstd is None:
    for cand in ("libzstd.so.1", ctypes.util.find_library("zstd")):
      if not cand:
        continue
      try:
        lib = ctypes.CDLL(cand)
        lib.ZSTD_getFrameContentSize.restype = ctypes.c_ulonglong
        lib.ZSTD_getFrameContentSize.argtypes = [ctypes.c_void_p, ctypes.c_size_t]
        lib.ZSTD_decompress.restype = ctypes.c_size_t
        lib.ZSTD_decompress.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_size_t]
        lib.ZSTD_isError.restype = ctypes.c_uint
        lib.ZSTD_isError.argtypes = [ctypes.c_size_t]
        _zstd = lib
        break
      except OSError:
        continue
    if _zstd is None:
      _zstd = False
  return _zstd


def zstd_decompress(data: bytes, max_out: Optional[int] = None) -> bytes:
  lib = _load_zstd()
  if not lib:
    raise RuntimeError("libzstd is not available; cannot read a zstd-compressed checkpoint")
  n = lib.ZSTD_getFrameContentSize(data, len(data))
  if n in (2**64 - 1, 2**64 - 2):   # unknown / error
    n = max_out or (len(data) * 64)
  out = ctypes.create_string_buffer(int(n))
  got = lib.ZSTD_decompress(out, int(n), data, len(data))
  if lib.ZSTD_isError(got):
    raise RuntimeError("zstd decompression failed")
  return out.raw[:got]


# ---------------------------------------------------------------------------- write
def _write_file(path: str, data: bytes) -> None:
  tmp = path + ".tmp"
  with open(tmp, "wb") as f:
    f.write(data)
  os.replace(tmp, path)


class _StoreWriter:
  """Collects what a process writes (array chunks, `.zarray` descriptors) and commits it as one OCDBT store under
  `ocdbt.process_<r>/` - the per-process layout Orbax uses before it merges manifests. Same interface as the
  native file writer pool (`submit`, `wait`, `close`)."""

  def __init__(self, directory: str, process_index: int):
    self.target = os.path.join(directory, f"ocdbt.process_{process_index}")
    self.root = directory
    self.items: Dict[str, bytes] = {}

  def submit(self, path: str, data: bytes) -> None:
    self.items[os.path.relpath(path, self.root).replace(os.sep, "/")] = bytes(data)

  def wait(self) -> None:
    from . import ocdbt
    if self.items:
      ocdbt.write_store(self.target, self.items)

  def close(self) -> None:
    self.items = {}


def write_tree(directory: str, tree: Mapping[Key, Any], process_index: int = 0,
               sharding_desc: Optional[Mapping[Key, Mapping[str, Any]]] = None, use_ocdbt: bool = False) -> None:
  """Writes `{key tuple: tensor | ShardedArray}` under `directory` in the Orbax plain-zarr layout, or - with
  `use_ocdbt` - with all array data of a process inside one OCDBT store `ocdbt.process_<r>/` (two files per
  process instead of two per array; `open_kv` reads the union of the stores).

  Called by every process of a job with the same keys. Plain tensors are replicated state: process 0
  writes them. A `ShardedArray` leaf is written by every process - its own chunk file - while process 0
  adds the array's `.zarray`. Process 0 also writes `_METADATA` / `_sharding`; each process its
  `array_metadatas/process_<r>`."""
  os.makedirs(directory, exist_ok=True)
  tree_md: Dict[str, Any] = {}
  arr_md: List[Dict[str, Any]] = []
  shard_md: Dict[str, str] = {}
  # array chunks go through the native writer pool (temp file + rename on worker threads)
  from ..runtime import native
  writer = _StoreWriter(directory, process_index) if use_ocdbt else native.AsyncWriter(threads=8)
  try:
    _write_tree_arrays(directory, tree, sharding_desc, writer, tree_md, arr_md, shard_md, process_index,
                       descriptor_sink=writer.submit if use_ocdbt else None)
    writer.wait()
  finally:
    writer.close()
  _write_tree_metadata(directory, process_index, tree_md, arr_md, shard_md)


def _write_tree_arrays(directory, tree, sharding_desc, writer, tree_md, arr_md, shard_md, process_index=0,
                       descriptor_sink=None) -> None:
  for key, t in tree.items():
    sharded = isinstance(t, ShardedArray)
    if not sharded and not isinstance(t, torch.Tensor):
      t = torch.as_tensor(t)
    name = param_name(key)
    pdir = os.path.join(directory, name)
    if sharded:
      data, zdtype, _ = _tensor_to_bytes(t.local)
      shape, chunks = list(t.global_shape), list(t.chunk_shape)
      if list(t.local.shape) != chunks:
        raise ValueError(f"{name}: local chunk {list(t.local.shape)} does not match chunk_shape {chunks}")
      chunk_name = ".".join(str(i) for i in t.chunk_index)
      sharding_type = "NamedSharding"
    else:
      data, zdtype, shape = _tensor_to_bytes(t)
      chunks = shape
      chunk_name = ".".join("0" for _ in shape) if shape else "0"
      sharding_type = "SingleDeviceSharding"
    if sharded or process_index == 0:
      if descriptor_sink is None:
        os.makedirs(pdir, exist_ok=True)
      writer.submit(os.path.join(pdir, chunk_name), data)
    if process_index == 0:
      zarray = {
          "chunks": chunks if chunks else [], "compressor": None, "dimension_separator": ".", "dtype": zdtype,
          "fill_value": None, "filters": None, "order": "C", "shape": shape, "zarr_format": 2,
      }
      if descriptor_sink is None:
        _write_file(os.path.join(pdir, ".zarray"), json.dumps(zarray).encode())
      else:
        descriptor_sink(os.path.join(pdir, ".zarray"), json.dumps(zarray).encode())
    tree_md[key_to_str(key)] = {
        "key_metadata": [{"key": str(k), "key_type": 1 if isinstance(k, int) else 2} for k in key],
        "value_metadata": {"value_type": "jax.Array", "skip_deserialize": False, "write_shape": chunks},
    }
    arr_md.append({"array_metadata": {"param_name": name, "write_shape": chunks, "chunk_shape": chunks,
                                      "ext_metadata": None}})
    desc = (sharding_desc or {}).get(key) or {"sharding_type": sharding_type, "device_str": "cuda:0"}
    shard_md[base64.b64encode(name.encode()).decode()] = json.dumps(desc)


def _write_tree_metadata(directory, process_index, tree_md, arr_md, shard_md) -> None:
  if process_index == 0:
    _write_file(os.path.join(directory, "_METADATA"), json.dumps({
        "tree_metadata": tree_md, "use_zarr3": False, "store_array_data_equal_to_fill_value": True,
        "custom_metadata": None}).encode())
    _write_file(os.path.join(directory, "_sharding"), json.dumps(shard_md).encode())
  os.makedirs(os.path.join(directory, "array_metadatas"), exist_ok=True)
  _write_file(os.path.join(directory, "array_metadatas", f"process_{process_index}"),
              json.dumps({"array_metadatas": arr_md}).encode())


# ---------------------------------------------------------------------------- read
def _parse_key_str(s: str, md: Mapping[str, Any]) -> Key:
  out: List[Union[str, int]] = []
  for k in md["key_metadata"]:
    out.append(int(k["key"]) if k.get("key_type") == 1 else k["key"])
  return tuple(out)


def read_tree_metadata(directory: str) -> Dict[Key, Dict[str, Any]]:
  with open(os.path.join(directory, "_METADATA")) as f:
    md = json.load(f)
  return {_parse_key_str(s, v): v for s, v in md["tree_metadata"].items()}


def _decode_chunk(raw: bytes, zarray: Mapping[str, Any], nbytes: int) -> bytes:
  comp = zarray.get("compressor")
  if comp is None:
    return raw
  cid = comp.get("id")
  if cid == "zstd":
    return zstd_decompress(raw, nbytes)
  if cid in ("zlib", "gzip"):
    import zlib
    return zlib.decompress(raw, 15 + (16 if cid == "gzip" else 0))
  raise RuntimeError(f"unsupported zarr compressor {cid!r}")


class _DirKV:
  """Key-value view of a plain directory (keys are relative paths)."""

  def __init__(self, root: str):
    self.root = root

  def get(self, key: str) -> Optional[bytes]:
    p = os.path.join(self.root, key)
    if not os.path.isfile(p):
      return None
    with open(p, "rb") as f:
      return f.read()


class _UnionKV:
  """Several stores read as one: the first that has a key answers (per-process stores hold disjoint keys)."""

  def __init__(self, stores):
    self.stores = list(stores)

  def get(self, key: str) -> Optional[bytes]:
    for store in self.stores:
      value = store.get(key)
      if value is not None:
        return value
    return None


def open_kv(directory: str):
  """Directory-backed store; the OCDBT store when `manifest.ocdbt` is present; the union of the per-process
  stores `ocdbt.process_<r>/` (plus loose files) when a checkpoint was written that way and never merged."""
  from . import ocdbt
  if os.path.exists(os.path.join(directory, "manifest.ocdbt")):
    return ocdbt.OcdbtStore(directory)
  per_process = sorted(d for d in (os.listdir(directory) if os.path.isdir(directory) else [])
                       if d.startswith("ocdbt.process_") and os.path.exists(os.path.join(directory, d, "manifest.ocdbt")))
  if per_process:
    return _UnionKV([ocdbt.OcdbtStore(os.path.join(directory, d)) for d in per_process] + [_DirKV(directory)])
  return _DirKV(directory)


def read_array(kv, name: str) -> torch.Tensor:
  zraw = kv.get(f"{name}/.zarray")
  if zraw is None:
    raise KeyError(name)
  zarray = json.loads(zraw)
  shape = list(zarray["shape"])
  chunks = list(zarray["chunks"]) or []
  zdtype = zarray["dtype"]
  sep = zarray.get("dimension_separator", ".")
  itemsize = 2 if zdtype == "bfloat16" else np.dtype(_NP_FROM_ZARR.get(zdtype, zdtype)).itemsize
  if not shape:
    raw = kv.get(f"{name}/0")
    if raw is None:
      return _bytes_to_tensor(b"\0" * itemsize, zdtype, [])
    return _bytes_to_tensor(_decode_chunk(raw, zarray, itemsize), zdtype, [])
  npd = np.int16 if zdtype == "bfloat16" else np.dtype(_NP_FROM_ZARR.get(zdtype, zdtype))
  out = np.zeros(shape, dtype=npd)
  grid = [max(1, -(-s // c)) for s, c in zip(shape, chunks)]
  for idx in np.ndindex(*grid):
    raw = kv.get(f"{name}/" + sep.join(str(i) for i in idx))
    if raw is None:
      continue   # chunk equal to the fill value
    nbytes = int(np.prod(chunks)) * itemsize
    buf = _decode_chunk(raw, zarray, nbytes)
    block = np.frombuffer(buf, dtype=npd).reshape(chunks)
    sl = tuple(slice(i * c, min((i + 1) * c, s)) for i, c, s in zip(idx, chunks, shape))
    out[sl] = block[tuple(slice(0, s.stop - s.start) for s in sl)]
  t = torch.from_numpy(out)
  return t.view(torch.bfloat16) if zdtype == "bfloat16" else t


def read_array_rows(kv, name: str, lo: int, hi: int) -> torch.Tensor:
  """Rows [lo, hi) along the first axis of a stored array, touching only the chunk files that hold them
  (how a rank reads its part of state that another job size wrote). Ranges past the end read as zeros."""
  zraw = kv.get(f"{name}/.zarray")
  if zraw is None:
    raise KeyError(name)
  zarray = json.loads(zraw)
  shape, chunks = list(zarray["shape"]), list(zarray["chunks"])
  zdtype = zarray["dtype"]
  sep = zarray.get("dimension_separator", ".")
  npd = np.int16 if zdtype == "bfloat16" else np.dtype(_NP_FROM_ZARR.get(zdtype, zdtype))
  itemsize = np.dtype(npd).itemsize
  out = np.zeros([hi - lo] + shape[1:], dtype=npd)
  c0 = chunks[0]
  rest_grid = [max(1, -(-s // c)) for s, c in zip(shape[1:], chunks[1:])]
  for i0 in range(lo // c0, min(-(-hi // c0), max(1, -(-shape[0] // c0)))):
    for idx in (np.ndindex(*rest_grid) if rest_grid else [()]):
      raw = kv.get(f"{name}/" + sep.join(str(i) for i in (i0,) + tuple(idx)))
      if raw is None:
        continue
      block = np.frombuffer(_decode_chunk(raw, zarray, int(np.prod(chunks)) * itemsize), dtype=npd).reshape(chunks)
      a, b = max(lo, i0 * c0), min(hi, (i0 + 1) * c0, shape[0])
      if b <= a:
        continue
      dst = (slice(a - lo, b - lo),) + tuple(slice(i * c, min((i + 1) * c, s))
                                              for i, c, s in zip(idx, chunks[1:], shape[1:]))
      src = (slice(a - i0 * c0, b - i0 * c0),) + tuple(slice(0, d.stop - d.start) for d in dst[1:])
      out[dst] = block[src]
  t = torch.from_numpy(out)
  return t.view(torch.bfloat16) if zdtype == "bfloat16" else t


def read_tree(directory: str, keys: Optional[Iterable[Key]] = None, partial: bool = False) -> Dict[Key, torch.Tensor]:
  """Reads arrays (all, or the requested keys). Missing keys raise KeyError unless `partial`."""
  md = read_tree_metadata(directory)
  kv = open_kv(directory)
  want = list(keys) if keys is not None else list(md.keys())
  out: Dict[Key, torch.Tensor] = {}
  for key in want:
    if key not in md:
      if partial:
        continue
      raise KeyError(f"{key} not found in checkpoint {directory}")
    out[key] = read_array(kv, param_name(key))
  return out


# ---------------------------------------------------------------------------- step directories
def write_checkpoint_metadata(step_dir: str, item_names: Sequence[str], custom_metadata: Optional[Mapping[str, Any]],
                              init_ns: int) -> None:
  handler = "orbax.checkpoint._src.handlers.standard_checkpoint_handler.StandardCheckpointHandler"
  md = {"item_handlers": {n: handler for n in item_names}, "metrics": {}, "performance_metrics": {},
        "init_timestamp_nsecs": init_ns, "commit_timestamp_nsecs": time.time_ns(),
        "custom_metadata": dict(custom_metadata or {})}
  _write_file(os.path.join(step_dir, "_CHECKPOINT_METADATA"), json.dumps(md).encode())


def read_checkpoint_metadata(step_dir: str) -> Dict[str, Any]:
  p = os.path.join(step_dir, "_CHECKPOINT_METADATA")
  if not os.path.exists(p):
    return {}
  with open(p) as f:
    return json.load(f)


def list_steps(root: str) -> List[int]:
  """Committed step directories (those with `_CHECKPOINT_METADATA`)."""
  if not root or not os.path.isdir(root):
    return []
  steps = []
  for n in os.listdir(root):
    if n.isdigit() and os.path.exists(os.path.join(root, n, "_CHECKPOINT_METADATA")):
      steps.append(int(n))
  return sorted(steps)
