"""Reader (and a minimal writer) for TensorStore's OCDBT key-value store, the container Orbax
puts zarr arrays in by default (`manifest.ocdbt` + `d/<id>` data files).

Format, as far as checkpoints use it:

* Every manifest and B+tree node is framed as `magic (4) | total length (u64 le) | version varint |
  compression (0 none, 1 zstd) | body | crc32c (4)`. Magics: manifest 0x0cdb3a2a, node 0x0cdb20de.
* Manifest body: uuid (16), manifest kind, max inline value bytes, max decoded node bytes
  (varints), version-tree arity log2 (u8), compression method (+ zstd level i32), then the
  versions stored inline: a data-file table, the number of versions, and column-wise arrays
  (generation, root height, root data-file id / offset / length, key / byte statistics, commit
  time u64), then the count of version-tree interior nodes (0 for checkpoints; deeper version
  trees are not followed).
* Data-file table: count, prefix lengths shared with the previous path (count - 1), suffix
  lengths, base-path lengths, then the suffix bytes. Paths are relative to the store directory.
* Node body: height (u8), data-file table, entry count, key prefix lengths (count - 1), key
  suffix lengths, for interior nodes the subtree common prefix lengths, the key suffix bytes;
  then for a leaf: value lengths, value kinds (0 inline, 1 out of line), data-file ids and
  offsets of the out-of-line values, and the inline bytes; for an interior node: child data-file
  ids, offsets, lengths and three statistics arrays. Keys inside a child omit the first
  `subtree common prefix` bytes of the key that led to it.

The reader is checked against a checkpoint written by Orbax (the tests read the reference's own
test checkpoint); out-of-line values and interior nodes are checked through the writer below.
"""
from __future__ import annotations

import os
import struct
from typing import Dict, Iterator, List, Optional, Sequence, Tuple

MANIFEST_MAGIC = bytes.fromhex("0cdb3a2a")
NODE_MAGIC = bytes.fromhex("0cdb20de")


class OcdbtError(ValueError):
  pass


# ---------------------------------------------------------------------------------------------
# crc32c (Castagnoli), table driven
# ---------------------------------------------------------------------------------------------
def _make_table():
  tbl = []
  for i in range(256):
    c = i
    for _ in range(8):
      c = (c >> 1) ^ 0x82F63B78 if c & 1 else c >> 1
    tbl.append(c)
  return tbl


_CRC_TABLE = _make_table()


def crc32c(data: bytes) -> int:
  c = 0xFFFFFFFF
  tbl = _CRC_TABLE
  for b in data:
    c = tbl[(c ^ b) & 0xFF] ^ (c >> 8)
  return c ^ 0xFFFFFFFF


# ---------------------------------------------------------------------------------------------
# byte cursor
# ---------------------------------------------------------------------------------------------
class _Cursor:

  def __init__(self, data: bytes):
    self.d = data
    self.i = 0

  def u8(self) -> int:
    v = self.d[self.i]
    self.i += 1
    return v

  def varint(self) -> int:
    shift = v = 0
    while True:
      if self.i >= len(self.d):
        raise OcdbtError("truncated varint")
      b = self.d[self.i]
      self.i += 1
      v |= (b & 0x7F) << shift
      if not b & 0x80:
        return v
      shift += 7
      if shift > 70:
        raise OcdbtError("varint too long")

  def varints(self, n: int) -> List[int]:
    return [self.varint() for _ in range(n)]

  def take(self, n: int) -> bytes:
    if self.i + n > len(self.d):
      raise OcdbtError("truncated field")
    out = self.d[self.i:self.i + n]
    self.i += n
    return out

  def u64s(self, n: int) -> List[int]:
    return list(struct.unpack("<" + "Q" * n, self.take(8 * n)))


def _unframe(blob: bytes, magic: bytes, verify: bool) -> bytes:
  if len(blob) < 18 or blob[:4] != magic:
    raise OcdbtError(f"bad magic {blob[:4].hex()} (want {magic.hex()})")
  (length,) = struct.unpack("<Q", blob[4:12])
  if length > len(blob) or length < 18:
    raise OcdbtError("frame length out of range")
  if verify and struct.unpack("<I", blob[length - 4:length])[0] != crc32c(blob[:length - 4]):
    raise OcdbtError("crc32c mismatch")
  cur = _Cursor(blob[:length - 4])
  cur.i = 12
  version = cur.varint()
  if version != 0:
    raise OcdbtError(f"unsupported format version {version}")
  comp = cur.varint()
  body = blob[cur.i:length - 4]
  if comp == 0:
    return body
  if comp == 1:
    from . import orbax_layout
    return orbax_layout.zstd_decompress(body)
  raise OcdbtError(f"unknown compression {comp}")


def _frame(magic: bytes, body: bytes) -> bytes:
  length = 4 + 8 + 1 + 1 + len(body) + 4
  head = magic + struct.pack("<Q", length) + b"\x00\x00" + body
  return head + struct.pack("<I", crc32c(head))


def _read_file_table(cur: _Cursor) -> List[str]:
  n = cur.varint()
  if n == 0:
    return []
  prefix = [0] + cur.varints(n - 1)
  suffix = cur.varints(n)
  cur.varints(n)                       # base-path lengths: a split point of the path, not needed
  paths, prev = [], b""
  for p, s in zip(prefix, suffix):
    cur_path = prev[:p] + cur.take(s)
    paths.append(cur_path.decode("utf-8"))
    prev = cur_path
  return paths


def _varint(v: int) -> bytes:
  out = bytearray()
  while True:
    b = v & 0x7F
    v >>= 7
    out.append(b | (0x80 if v else 0))
    if not v:
      return bytes(out)


def _write_file_table(paths: Sequence[str]) -> bytes:
  out = _varint(len(paths))
  if not paths:
    return out
  enc = [p.encode("utf-8") for p in paths]
  prefs = []
  for a, b in zip(enc, enc[1:]):
    k = 0
    while k < min(len(a), len(b)) and a[k] == b[k]:
      k += 1
    prefs.append(k)
  out += b"".join(_varint(k) for k in prefs)
  sufs = [enc[0]] + [b[k:] for b, k in zip(enc[1:], prefs)]
  out += b"".join(_varint(len(s)) for s in sufs)
  out += b"".join(_varint(0) for _ in enc)
  return out + b"".join(sufs)


# ---------------------------------------------------------------------------------------------
# reader
# ---------------------------------------------------------------------------------------------
class OcdbtStore:
  """Read-only view of the latest version of an OCDBT store: `get(key)`, `keys()`, `items()`."""

  def __init__(self, directory: str, verify_checksums: bool = True):
    self.dir = directory
    self._verify = verify_checksums
    with open(os.path.join(directory, "manifest.ocdbt"), "rb") as f:
      body = _unframe(f.read(), MANIFEST_MAGIC, verify_checksums)
    cur = _Cursor(body)
    self.uuid = cur.take(16)
    kind = cur.varint()
    if kind != 0:
      raise OcdbtError(f"manifest kind {kind} (numbered manifests) is not supported")
    self.max_inline_value_bytes = cur.varint()
    self.max_decoded_node_bytes = cur.varint()
    self.version_tree_arity_log2 = cur.u8()
    if cur.varint() == 1:
      cur.take(4)                      # zstd level
    files = _read_file_table(cur)
    n = cur.varint()
    if n == 0:
      self._root = None
      self._index: Optional[Dict[str, tuple]] = {}
      return
    gens = cur.varints(n)
    heights = [cur.u8() for _ in range(n)]
    fids, offs, lens = cur.varints(n), cur.varints(n), cur.varints(n)
    cur.varints(n); cur.varints(n); cur.varints(n)      # key / tree-byte / indirect-byte statistics
    cur.u64s(n)                                         # commit times
    if cur.i < len(body) and cur.varint() != 0:
      raise OcdbtError("version trees with interior nodes are not supported")
    latest = max(range(n), key=lambda i: gens[i])
    self.generation = gens[latest]
    self._root = (files[fids[latest]], offs[latest], lens[latest], heights[latest])
    self._index = None
    self._files: Dict[str, bytes] = {}

  # -- low level -------------------------------------------------------------------------------
  def _read(self, path: str, offset: int, length: int) -> bytes:
    with open(os.path.join(self.dir, path), "rb") as f:
      f.seek(offset)
      data = f.read(length)
    if len(data) != length:
      raise OcdbtError(f"{path}: wanted {length} bytes at {offset}, file is shorter")
    return data

  def _walk(self, loc, prefix: bytes) -> Iterator[Tuple[bytes, tuple]]:
    path, off, length, want_height = loc
    cur = _Cursor(_unframe(self._read(path, off, length), NODE_MAGIC, self._verify))
    height = cur.u8()
    if height != want_height:
      raise OcdbtError(f"node height {height}, parent says {want_height}")
    files = _read_file_table(cur)
    n = cur.varint()
    if n == 0:
      return
    pre = [0] + cur.varints(n - 1)
    suf = cur.varints(n)
    common = cur.varints(n) if height > 0 else None
    keys, prev = [], b""
    for p, s in zip(pre, suf):
      k = prev[:p] + cur.take(s)
      keys.append(k)
      prev = k
    if height == 0:
      vlen = cur.varints(n)
      kinds = [cur.u8() for _ in range(n)]
      n_out = sum(1 for k in kinds if k == 1)
      fids, offs = cur.varints(n_out), cur.varints(n_out)
      j = 0
      for key, ln, kind in zip(keys, vlen, kinds):
        if kind == 0:
          yield prefix + key, ("inline", cur.take(ln))
        elif kind == 1:
          yield prefix + key, ("file", files[fids[j]], offs[j], ln)
          j += 1
        else:
          raise OcdbtError(f"unknown value kind {kind}")
      return
    fids, offs, lens = cur.varints(n), cur.varints(n), cur.varints(n)
    for i, key in enumerate(keys):
      child = (files[fids[i]], offs[i], lens[i], height - 1)
      yield from self._walk(child, prefix + key[:common[i]])

  def _build(self) -> Dict[str, tuple]:
    if self._index is None:
      self._index = {}
      if self._root is not None:
        for k, ref in self._walk(self._root, b""):
          self._index[k.decode("utf-8")] = ref
    return self._index

  # -- key-value interface -----------------------------------------------------------------------
  def keys(self) -> List[str]:
    return sorted(self._build())

  def get(self, key: str) -> Optional[bytes]:
    ref = self._build().get(key)
    if ref is None:
      return None
    if ref[0] == "inline":
      return ref[1]
    return self._read(ref[1], ref[2], ref[3])

  def items(self) -> Iterator[Tuple[str, bytes]]:
    for k in self.keys():
      yield k, self.get(k)


# ---------------------------------------------------------------------------------------------
# writer (single version; values above `max_inline` go to one data file; optional 2-level tree)
# ---------------------------------------------------------------------------------------------
def _encode_keys(keys: Sequence[bytes]) -> Tuple[bytes, bytes, bytes]:
  prefs, sufs = [], [keys[0]]
  for a, b in zip(keys, keys[1:]):
    k = 0
    while k < min(len(a), len(b)) and a[k] == b[k]:
      k += 1
    prefs.append(k)
    sufs.append(b[k:])
  return (b"".join(_varint(k) for k in prefs), b"".join(_varint(len(s)) for s in sufs), b"".join(sufs))


def write_store(directory: str, items: Dict[str, bytes], max_inline: int = 100, leaf_size: int = 0,
                data_file: str = "d/00000000000000000000000000000001") -> None:
  """Writes `items` as one version. `leaf_size > 0` splits the keys over several leaves under one
  interior root (keys in a leaf drop the prefix common to that leaf). Uncompressed frames."""
  os.makedirs(os.path.join(directory, os.path.dirname(data_file)), exist_ok=True)
  keys = sorted(items)
  blob = bytearray()

  def put(b: bytes) -> Tuple[int, int]:
    off = len(blob)
    blob.extend(b)
    return off, len(b)

  refs = {}
  for k in keys:
    if len(items[k]) > max_inline:
      refs[k] = put(items[k])

  def leaf(sub: Sequence[str], strip: int) -> bytes:
    kb = [k.encode("utf-8")[strip:] for k in sub]
    pre, suf, raw = _encode_keys(kb)
    out = bytes([0]) + _write_file_table([data_file]) + _varint(len(sub)) + pre + suf + raw
    out += b"".join(_varint(len(items[k])) for k in sub)
    out += bytes(1 if k in refs else 0 for k in sub)
    outs = [k for k in sub if k in refs]
    out += b"".join(_varint(0) for _ in outs) + b"".join(_varint(refs[k][0]) for k in outs)
    out += b"".join(items[k] for k in sub if k not in refs)
    return _frame(NODE_MAGIC, out)

  if not leaf_size or len(keys) <= leaf_size:
    root_off, root_len = put(leaf(keys, 0)) if keys else (0, 0)
    height = 0
  else:
    groups = [keys[i:i + leaf_size] for i in range(0, len(keys), leaf_size)]
    entries = []
    for g in groups:
      enc = [k.encode("utf-8") for k in g]
      common = os.path.commonprefix(enc)
      off, ln = put(leaf(g, len(common)))
      entries.append((enc[0], len(common), off, ln, len(g)))
    pre, suf, raw = _encode_keys([e[0] for e in entries])
    out = bytes([1]) + _write_file_table([data_file]) + _varint(len(entries)) + pre + suf
    out += b"".join(_varint(e[1]) for e in entries) + raw
    out += b"".join(_varint(0) for _ in entries) + b"".join(_varint(e[2]) for e in entries)
    out += b"".join(_varint(e[3]) for e in entries) + b"".join(_varint(e[4]) for e in entries)
    out += b"".join(_varint(e[3]) for e in entries) + b"".join(_varint(0) for _ in entries)
    root_off, root_len = put(_frame(NODE_MAGIC, out))
    height = 1
  with open(os.path.join(directory, data_file), "wb") as f:
    f.write(bytes(blob))
  body = bytes(16) + _varint(0) + _varint(max_inline) + _varint(8 << 20) + bytes([4]) + _varint(0)
  body += _write_file_table([data_file])
  if keys:
    body += _varint(1) + _varint(1) + bytes([height]) + _varint(0) + _varint(root_off) + _varint(root_len)
    body += _varint(len(keys)) + _varint(root_len) + _varint(sum(v[1] for v in refs.values())) + struct.pack("<Q", 0)
  else:
    body += _varint(0)
  body += _varint(0)
  with open(os.path.join(directory, "manifest.ocdbt"), "wb") as f:
    f.write(_frame(MANIFEST_MAGIC, body))
