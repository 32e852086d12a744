"""tx_rmsnorm_bwd_static: the RMSNorm backward whose scratch is a device array inside the
library. Called through its exported C symbol, compared with tx_rmsnorm_bwd on two calls in
a row, and checked for the size limit. Collected last so that it also runs after every other
test has used the device."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
  from tunix_b200.ops import _lib
  lib = ctypes.CDLL(str(_lib.lib_path()))   # same image as the one the package loaded
  P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
  fn = lib.tx_rmsnorm_bwd_static
  fn.argtypes = [P, P, P, P, P, P, P, I, I, I, F, F, P]
  fn.restype = I
  lib.tx_rmsnorm_bwd_static_max_d.argtypes = []
  lib.tx_rmsnorm_bwd_static_max_d.restype = I
  lib.tx_rmsnorm_bwd_static_strerror.argtypes = [I]
  lib.tx_rmsnorm_bwd_static_strerror.restype = ctypes.c_char_p
  return lib


def _call(lib, x, w, dy, rstd, dres, dx, dw, accumulate, eps, offset):
  T, D = x.shape
  return lib.tx_rmsnorm_bwd_static(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(),
                                   dres.data_ptr() if dres is not None else None, dx.data_ptr(), dw.data_ptr(),
                                   int(accumulate), T, D, eps, offset, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("T,D", [(37, 256), (1000, 4096)])
def test_static_scratch_matches_existing_entry_point(kernel_lib, T, D):
  from tunix_b200.ops import kernels
  lib = _symbols()
  assert lib.tx_rmsnorm_bwd_static_max_d() == 4096
  dev = torch.device("cuda", torch.cuda.current_device())
  eps, offset = 1e-6, 0.0
  g = torch.Generator(device=dev).manual_seed(5)
  w = (1 + 0.1 * torch.randn(D, device=dev, generator=g)).bfloat16()
  for call in range(2):   # the second call reuses the scratch that the first one left dirty
    x = torch.randn(T, D, device=dev, generator=g).bfloat16()
    dy = torch.randn(T, D, device=dev, generator=g).bfloat16()
    dres = torch.randn(T, D, device=dev, generator=g).bfloat16()
    _, _, rstd = kernels.rmsnorm_fwd(x, w, eps, offset)
    dx_ref, dw_ref = kernels.rmsnorm_bwd(x, w, dy, rstd, eps, offset, dres=dres)
    dx = torch.empty_like(x)
    dw = torch.full((D,), float("nan"), dtype=torch.float32, device=dev)
    torch.cuda.synchronize()
    before = torch.cuda.memory_stats(dev)["allocation.all.allocated"]
    rc = _call(lib, x, w, dy, rstd, dres, dx, dw, False, eps, offset)
    assert rc == 0, lib.tx_rmsnorm_bwd_static_strerror(rc).decode()
    torch.cuda.synchronize()
    assert torch.cuda.memory_stats(dev)["allocation.all.allocated"] == before
    torch.testing.assert_close(dx.float(), dx_ref.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(dw, dw_ref, rtol=1e-5, atol=1e-4)
    # accumulate into an existing dw
    rc = _call(lib, x, w, dy, rstd, None, dx, dw, True, eps, offset)
    assert rc == 0
    torch.cuda.synchronize()
    torch.testing.assert_close(dw, 2 * dw_ref, rtol=1e-5, atol=2e-4)


def test_static_scratch_rejects_oversize(kernel_lib):
  lib = _symbols()
  dev = torch.device("cuda", torch.cuda.current_device())
  T, D = 4, 8192
  x = torch.zeros(T, D, device=dev, dtype=torch.bfloat16)
  w = torch.ones(D, device=dev, dtype=torch.bfloat16)
  rstd = torch.ones(T, device=dev)
  dx = torch.full_like(x, 3.0)
  dw = torch.full((D,), 7.0, device=dev)
  rc = _call(lib, x, w, x, rstd, None, dx, dw, False, 1e-6, 0.0)
  assert rc == 2
  assert b"4096" in lib.tx_rmsnorm_bwd_static_strerror(rc)
  torch.cuda.synchronize()
  assert float(dx.float().min()) == 3.0 and float(dw.min()) == 7.0   # nothing was launched
  x12 = torch.zeros(T, 12, device=dev, dtype=torch.bfloat16)
  assert _call(lib, x12, w, x12, rstd, None, x12.clone(), dw, False, 1e-6, 0.0) == 1
