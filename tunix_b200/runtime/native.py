"""ctypes bindings of `csrc/host_runtime.cc` (linked into the kernel library).

Every function has a plain-Python equivalent that is used when the library has not been built,
so callers never need to check: `ffd_pack`, `read_into` (parallel positional read into a
buffer), `AsyncWriter` (write-to-temp + rename on worker threads).
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import List, Optional, Sequence

import numpy as np

_lib = None
_checked = False


def _native():
  global _lib, _checked
  if not _checked:
    _checked = True
    try:
      from ..ops import _lib as kernel_lib
      lib = kernel_lib.load()
      if lib is not None and hasattr(lib, "tx_ffd_pack"):
        lib.tx_ffd_pack.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_longlong, ctypes.c_int,
                                    ctypes.c_void_p]
        lib.tx_ffd_pack.restype = ctypes.c_int
        lib.tx_pread_parallel.argtypes = [ctypes.c_char_p, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_void_p,
                                          ctypes.c_int]
        lib.tx_pread_parallel.restype = ctypes.c_int
        lib.tx_writer_create.argtypes = [ctypes.c_int]
        lib.tx_writer_create.restype = ctypes.c_void_p
        lib.tx_writer_submit.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_void_p, ctypes.c_longlong,
                                         ctypes.c_int]
        lib.tx_writer_submit.restype = ctypes.c_int
        lib.tx_writer_wait.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int)]
        lib.tx_writer_wait.restype = ctypes.c_int
        lib.tx_writer_destroy.argtypes = [ctypes.c_void_p]
        lib.tx_writer_destroy.restype = None
        _lib = lib
    except Exception:  # pylint: disable=broad-exception-caught
      _lib = None
  return _lib


def available() -> bool:
  return _native() is not None


def ffd_pack_py(lengths: Sequence[int], pack_size: int, budget: int, max_segments: int) -> List[int]:
  assign = [-1] * len(lengths)
  loads, counts = [0] * pack_size, [0] * pack_size
  for i in sorted(range(len(lengths)), key=lambda j: lengths[j], reverse=True):
    for b in range(pack_size):
      if loads[b] + lengths[i] <= budget and counts[b] < max_segments:
        assign[i] = b
        loads[b] += lengths[i]
        counts[b] += 1
        break
  return assign


def ffd_pack(lengths: Sequence[int], pack_size: int, budget: int, max_segments: int) -> List[int]:
  """First-fit-decreasing: bin index per item (input order), -1 for items that fit nowhere."""
  lib = _native()
  n = len(lengths)
  if lib is None or n == 0:
    return ffd_pack_py(lengths, pack_size, budget, max_segments)
  arr = np.ascontiguousarray(lengths, dtype=np.int32)
  out = np.empty(n, dtype=np.int32)
  rc = lib.tx_ffd_pack(arr.ctypes.data, n, int(pack_size), int(budget), int(max_segments), out.ctypes.data)
  if rc != 0:
    raise ValueError(f"tx_ffd_pack rejected its arguments (code {rc})")
  return out.tolist()


def read_into(path: str, offset: int, nbytes: int, dst_ptr: int, threads: int = 8) -> None:
  """Reads `nbytes` at `offset` of `path` into memory at `dst_ptr` (e.g. a pinned tensor's data_ptr)."""
  lib = _native()
  if lib is not None:
    rc = lib.tx_pread_parallel(os.fsencode(path), int(offset), int(nbytes), ctypes.c_void_p(dst_ptr), int(threads))
    if rc != 0:
      raise OSError(rc, os.strerror(rc), path)
    return
  buf = (ctypes.c_char * nbytes).from_address(dst_ptr)
  with open(path, "rb") as f:
    f.seek(offset)
    got = f.readinto(buf)
  if got != nbytes:
    raise OSError(f"{path}: wanted {nbytes} bytes at {offset}, got {got}")


class AsyncWriter:
  """`submit(path, buffer)` returns at once; `wait()` blocks until everything is on disk and raises if a
  write failed. Buffers (bytes, NumPy arrays, CPU tensors) are kept alive until then."""

  def __init__(self, threads: int = 4, fsync: bool = False):
    self._fsync = fsync
    self._keep: List[object] = []
    self._lock = threading.Lock()
    lib = _native()
    self._lib = lib
    self._h = lib.tx_writer_create(int(threads)) if lib is not None else None
    self._py_threads: List[threading.Thread] = []
    self._py_errors: List[BaseException] = []

  @staticmethod
  def _view(buf):
    if isinstance(buf, (bytes, bytearray, memoryview)):
      mv = memoryview(buf)
      arr = np.frombuffer(mv, dtype=np.uint8)
      return arr, arr.ctypes.data, arr.nbytes
    if isinstance(buf, np.ndarray):
      arr = np.ascontiguousarray(buf)
      return arr, arr.ctypes.data, arr.nbytes
    if hasattr(buf, "data_ptr"):       # torch CPU tensor
      t = buf.contiguous()
      return t, t.data_ptr(), t.numel() * t.element_size()
    raise TypeError(f"cannot write a {type(buf).__name__}")

  def submit(self, path: str, buf) -> None:
    keep, ptr, n = self._view(buf)
    with self._lock:
      self._keep.append(keep)
    if self._h is not None:
      rc = self._lib.tx_writer_submit(self._h, os.fsencode(path), ctypes.c_void_p(ptr), n, int(self._fsync))
      if rc != 0:
        raise OSError(rc, os.strerror(rc), path)
      return

    def work():
      try:
        tmp = f"{path}.tmp.{threading.get_ident()}"
        with open(tmp, "wb") as f:
          f.write((ctypes.c_char * n).from_address(ptr) if n else b"")
          if self._fsync:
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
      except BaseException as e:  # pylint: disable=broad-exception-caught
        self._py_errors.append(e)
    t = threading.Thread(target=work, daemon=True)
    t.start()
    self._py_threads.append(t)

  def wait(self) -> None:
    if self._h is not None:
      first = ctypes.c_int(0)
      failed = self._lib.tx_writer_wait(self._h, ctypes.byref(first))
      with self._lock:
        self._keep.clear()
      if failed:
        raise OSError(first.value, f"{failed} asynchronous write(s) failed: {os.strerror(first.value)}")
      return
    for t in self._py_threads:
      t.join()
    self._py_threads.clear()
    with self._lock:
      self._keep.clear()
    if self._py_errors:
      e = self._py_errors[0]
      self._py_errors.clear()
      raise OSError(f"asynchronous write failed: {e}")

  def close(self) -> None:
    if self._h is not None:
      try:
        self.wait()
      finally:
        self._lib.tx_writer_destroy(self._h)
        self._h = None

  def __del__(self):
    try:
      if self._h is not None:
        self._lib.tx_writer_destroy(self._h)
        self._h = None
    except Exception:  # pylint: disable=broad-exception-caught
      pass
