"""ctypes loader for the in-tree sm_100a kernel library.

The library is plain C ABI (no torch headers); tensors cross as raw device pointers plus
the current CUDA stream. On a machine with a GPU a missing library is an error, never a
silent fallback: `require()` raises with the build command.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIB = None
_LOCK = threading.Lock()
_DEBUG_KERNELS = os.environ.get("TUNIX_B200_DEBUG_KERNELS", "0") == "1"     # the -DTX_DEBUG build (index checks)
_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / (
    "libtunix_b200_debug.so" if _DEBUG_KERNELS else "libtunix_b200.so")

c_void_p = ctypes.c_void_p
c_int = ctypes.c_int
c_ll = ctypes.c_longlong
c_float = ctypes.c_float


def lib_path() -> Path:
  return _LIB_PATH


def available() -> bool:
  """True when the compiled library exists and a CUDA device is usable."""
  return _LIB_PATH.exists() and torch.cuda.is_available()


def _declare(lib):
  P, I, L, F = c_void_p, c_int, c_ll, c_float
  sigs = {
      "tx_gemm_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, I, F, P, I, P],
      "tx_rmsnorm_fwd": [P, P, P, P, P, P, I, I, F, F, P],
      "tx_rmsnorm_bwd_partials": [I],
      "tx_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, I, I, F, F, P],
      "tx_qknorm_rope_fwd": [P, P, P, P, P, P, P, L, I, I, I, I, L, L, F, F, I, I, P, P, P, P, P],
      "tx_qknorm_rope_bwd": [P, P, P, P, P, P, P, P, P, L, I, I, I, I, L, L, L, F, F, I, P, P],
      "tx_glu_fwd": [P, P, L, I, I, P],
      "tx_glu_bwd": [P, P, P, L, I, I, P],
      "tx_embedding_fwd": [P, P, P, L, I, I, F, P],
      "tx_embedding_bwd": [P, P, P, L, I, I, F, P],
      "tx_adamw": [P, P, P, P, P, L, F, F, F, F, F, F, F, P, I, P],
      "tx_sumsq_partials": [],
      "tx_sumsq": [P, L, P, P, I, P],
      "tx_clip_scale": [P, P, F, P, P, P],
      "tx_cast_f32_bf16": [P, P, L, P],
      "tx_accum_bf16_f32": [P, P, L, F, P],
      "tx_flash_fwd": [P, P, P, P, P, I, I, I, I, I, I, L, L, L, L, I, F, P, P],
      "tx_flash_bwd": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, L, L, L, L, L, L, L, L, I, F, P, P],
      "tx_flash_fwd_seg": [P, P, P, P, P, I, I, I, I, I, I, L, L, L, L, I, F, P, P, P, P],
      "tx_flash_bwd_seg": [P, P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, L, L, L, L, L, L, L, L, I, F, P, P, P, P],
      "tx_gemm_bf16_dual": [P, P, P, P, P, I, I, I, I, L, L, L, L, L, I, I, I, I, F, P, I, P],
      "tx_gemm_grouped_bf16": [P, P, P, P, P, I, I, I, I, I, L, L, L, I, I, F, P, P],
      "tx_moe_dispatch_rows": [P, L, P, I, P, P, P, ctypes.POINTER(P), I, L, I, L, P, P],
      "tx_moe_combine_rows": [ctypes.POINTER(P), I, P, P, P, I, P, L, P, L, I, L, P, P],
      "tx_gemm_bf16_allgather_b": [P, ctypes.POINTER(P), I, I, P, P, P, I, I, I, L, L, L, I, I, F, L, P, P],
      "tx_gemm_bf16_allreduce": [P, P, ctypes.POINTER(P), I, I, I, I, L, L, I, I, F, P, P],
      "tx_f32_sum_to_bf16": [P, P, L, I, I, P],
      "tx_kv_page_write": [P, P, L, L, P, P, P, I, I, I, P],
      "tx_paged_decode_attn": [P, L, P, P, P, I, P, I, I, I, I, I, F, I, P, P, P, L, P],
      "tx_paged_decode_attn_tc": [P, L, P, P, P, I, P, I, I, I, I, I, L, F, I, P, P, P, L, P, P],
      "tx_paged_decode_combine": [P, P, I, P, L, I, I, I, P],
      "tx_peer_barrier": [ctypes.POINTER(P), I, I, I, L, P, P],
      "tx_reduce_scatter_grid": [],
      "tx_reduce_scatter_sum_f32": [ctypes.POINTER(P), P, L, L, I, I, P, P],
      "tx_adamw_allgather": [P, P, P, P, ctypes.POINTER(P), L, L, F, F, F, F, F, F, F, P, I, I, P],
      "tx_peer_copy_2d": [P, P, L, L, L, L, P],
      "tx_sample": [P, I, L, I, I, F, I, ctypes.c_ulonglong, P, L, P, I, P, P, P],
      "tx_sample_filtered": [P, I, L, I, I, F, I, F, ctypes.c_ulonglong, P, L, P, I, P, P, P],
      "tx_gemm_skinny_flag_blocks": [],
      "tx_gemm_skinny_set_pdl": [I],
      "tx_gemm_skinny": [P, P, P, P, P, I, I, I, L, L, L, L, F, I, I, P, I, I, I, ctypes.POINTER(P),
                         ctypes.POINTER(P), L, P, P, L, P],
      "tx_logprob_fwd": [P, I, L, P, P, P, P, I, I, F, F, P],
      "tx_logprob_bwd": [P, I, L, P, P, P, P, P, P, L, I, I, I, F, F, P],
  }
  for name, argtypes in sigs.items():
    fn = getattr(lib, name, None)
    if fn is None:
      continue
    fn.argtypes = argtypes
    fn.restype = c_int
  return lib


def declare(name: str, argtypes, restype=c_int):
  """Registers the signature of an additional exported symbol (used by optional modules)."""
  lib = require()
  fn = getattr(lib, name)
  fn.argtypes = argtypes
  fn.restype = restype
  return fn


def load():
  """Returns the ctypes library or None when it has not been built."""
  global _LIB
  if _LIB is not None:
    return _LIB
  with _LOCK:
    if _LIB is None and _LIB_PATH.exists():
      _LIB = _declare(ctypes.CDLL(str(_LIB_PATH), mode=ctypes.RTLD_GLOBAL))
      if _DETERMINISTIC and hasattr(_LIB, "tx_gemm_set_deterministic"):
        _LIB.tx_gemm_set_deterministic(1)
  return _LIB


_DETERMINISTIC = os.environ.get("TUNIX_B200_DETERMINISTIC", "0") == "1"


def deterministic() -> bool:
  return _DETERMINISTIC


def set_deterministic(flag: bool) -> None:
  """Bitwise-reproducible mode (also `TUNIX_B200_DETERMINISTIC=1`): products whose partial sums would meet through
  floating-point atomics take their single-pass form - no split-K in skinny GEMMs, and tensor-parallel exits
  all-reduce through the collective library instead of the atomic-add epilogue. Flash attention (fixed reduction
  order), the log-prob kernels, the grouped expert GEMMs and the Philox sampler are reproducible in either mode;
  the embedding gradient switches from fp32 atomic adds to a sorted accumulation."""
  global _DETERMINISTIC
  _DETERMINISTIC = bool(flag)
  lib = load()
  if lib is not None and hasattr(lib, "tx_gemm_set_deterministic"):
    lib.tx_gemm_set_deterministic(int(_DETERMINISTIC))


def require():
  lib = load()
  if lib is None:
    raise RuntimeError(
        f"{_LIB_PATH} is missing. Build it with `python -m tunix_b200.build_kernels` "
        "(needs nvcc); CUDA tensors cannot be processed without the sm_100a kernels.")
  return lib


_HOME_DEVICE = None    # one process drives one GPU: the device current when the first kernel is launched


def bind_thread() -> None:
  """Makes this host thread use the process's GPU.

  The CUDA current device is per thread and starts at 0, so a helper thread of rank r (a rollout
  producer, an asyncio loop) would otherwise launch on GPU 0 with pointers that live on GPU r."""
  global _HOME_DEVICE
  cur = torch.cuda.current_device()
  if _HOME_DEVICE is None:
    _HOME_DEVICE = cur
  elif cur != _HOME_DEVICE:
    torch.cuda.set_device(_HOME_DEVICE)


def stream_ptr() -> int:
  bind_thread()
  return torch.cuda.current_stream().cuda_stream


_status = {}


def status_word(device) -> torch.Tensor:
  """Per-device int32 word that kernels OR error bits into (bounded waits that gave up...)."""
  key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
  t = _status.get(key)
  if t is None:
    t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    _status[key] = t
  return t


def check_status(device=None) -> None:
  """Synchronising check of the kernel status word; raises if any kernel reported an error."""
  if not torch.cuda.is_available():
    return
  dev = torch.cuda.current_device() if device is None else torch.device(device).index
  t = _status.get(dev)
  if t is None:
    return
  v = int(t.item())
  _check_debug_records()
  if v != 0:
    t.zero_()
    raise RuntimeError(f"tunix_b200 kernel reported error status 0x{v:x} "
                       "(1/2/4: producer/MMA/epilogue wait timed out, 8: bad argument, 16: peer wait timed out)")


_DEBUG_UNITS = ("elementwise", "logprob")
_DEBUG_CODES = {1: "token id outside the vocabulary (embedding)", 2: "target id outside the vocabulary (log-prob)",
                3: "block-table page outside the cache (paged attention)", 4: "slot beyond the cache (KV page write)"}


def _check_debug_records() -> None:
  """Debug build only: raises when a kernel recorded an index that the release build would have resolved silently."""
  lib = _LIB
  if lib is None or not _DEBUG_KERNELS:
    return
  for unit in _DEBUG_UNITS:
    fn = getattr(lib, f"tx_debug_read_{unit}", None)
    if fn is None:
      continue
    rec = (ctypes.c_int * 4)()
    fn.argtypes, fn.restype = [ctypes.POINTER(ctypes.c_int)], ctypes.c_int
    if fn(rec) > 0:
      raise RuntimeError(f"debug kernels ({unit}): {_DEBUG_CODES.get(rec[1], rec[1])}: value {rec[2]}, limit {rec[3]}")


launch_calls = 0   # number of library launches issued by this process (each is >= 1 kernel)


def check_rc(rc: int, what: str) -> None:
  global launch_calls
  launch_calls += 1
  if rc != 0:
    raise RuntimeError(f"{what} failed with code {rc}")
