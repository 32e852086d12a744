"""Builds the sm_100a CUDA library in-tree with plain nvcc (no torch headers needed).

Every ``.cu`` under ``tunix_b200/csrc`` is compiled to an object file and linked into
``tunix_b200/lib/libtunix_b200.so``; the Python side loads it with ctypes. The C++-only
runtime pieces (``.cc``) are linked into the same library.

Usage: ``python -m tunix_b200.build_kernels [--force] [--verbose] [--debug]``

``--debug`` builds ``libtunix_b200_debug.so`` from the same sources with ``-DTX_DEBUG``: kernels then record
index errors that the release build resolves silently (``csrc/tx_debug.cuh``). Load it with
``TUNIX_B200_DEBUG_KERNELS=1``.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB_DIR = PKG / "lib"
BUILD_DIR = PKG / "lib" / "obj"
LIB_PATH = LIB_DIR / "libtunix_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-O3",
]


def find_nvcc() -> str:
  cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
  if not Path(cand).exists():
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")
  return cand


def _digest(paths) -> str:
  h = hashlib.sha256()
  for p in sorted(paths):
    h.update(str(p).encode())
    h.update(Path(p).read_bytes())
  h.update(" ".join(NVCC_FLAGS).encode())
  return h.hexdigest()


def sources():
  return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cc")))


def headers():
  return sorted(list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")))


DEBUG_LIB_PATH = LIB_DIR / "libtunix_b200_debug.so"
DEBUG_BUILD_DIR = PKG / "lib" / "obj_debug"


def _compile_one(nvcc: str, src: Path, verbose: bool, ptxas_info: bool, debug: bool = False) -> Path:
  bdir = DEBUG_BUILD_DIR if debug else BUILD_DIR
  obj = bdir / (src.stem + ".o")
  stamp = bdir / (src.stem + ".sha")
  want = _digest([src] + headers()) + ("-debug" if debug else "")
  if obj.exists() and stamp.exists() and stamp.read_text() == want:
    return obj
  cmd = [nvcc] + NVCC_FLAGS + ["-I", str(CSRC), "-c", str(src), "-o", str(obj)]
  if src.suffix == ".cc":
    cmd = [nvcc] + NVCC_FLAGS + ["-x", "cu", "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
  if ptxas_info:
    cmd += ["-Xptxas", "-v"]
  if debug:
    cmd += ["-DTX_DEBUG"]
  if verbose:
    print(" ".join(cmd), flush=True)
  r = subprocess.run(cmd, capture_output=True, text=True)
  if r.returncode != 0:
    raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
  if ptxas_info or verbose:
    sys.stderr.write(r.stderr)
  stamp.write_text(want)
  return obj


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False, debug: bool = False) -> Path:
  """Compiles (if stale) and links the library (the `-DTX_DEBUG` one with `debug`); returns its path."""
  nvcc = find_nvcc()
  bdir, lib = (DEBUG_BUILD_DIR, DEBUG_LIB_PATH) if debug else (BUILD_DIR, LIB_PATH)
  LIB_DIR.mkdir(exist_ok=True)
  bdir.mkdir(exist_ok=True)
  if force:
    for f in bdir.glob("*.sha"):
      f.unlink()
  srcs = sources()
  lib_stamp = bdir / "lib.sha"
  want = _digest(srcs + headers())
  if lib.exists() and lib_stamp.exists() and lib_stamp.read_text() == want and not force:
    return lib
  with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(srcs)))) as ex:
    objs = list(ex.map(lambda s: _compile_one(nvcc, s, verbose, ptxas_info, debug), srcs))
  cmd = [nvcc, "-shared", "-o", str(lib)] + [str(o) for o in objs] + ["-lcudart", "-lpthread", "-ldl"]
  if verbose:
    print(" ".join(cmd), flush=True)
  r = subprocess.run(cmd, capture_output=True, text=True)
  if r.returncode != 0:
    raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
  lib_stamp.write_text(want)
  return lib


def main(argv=None):
  ap = argparse.ArgumentParser()
  ap.add_argument("--force", action="store_true")
  ap.add_argument("--verbose", action="store_true")
  ap.add_argument("--ptxas-info", action="store_true")
  ap.add_argument("--debug", action="store_true", help="build the index-checking library (-DTX_DEBUG)")
  a = ap.parse_args(argv)
  p = build(a.force, a.verbose, a.ptxas_info, a.debug)
  print(p)


if __name__ == "__main__":
  main()
