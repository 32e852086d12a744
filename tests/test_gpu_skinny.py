"""The stream-K skinny (decode) GEMM against fp32 PyTorch: plain, gated, residual / bias epilogues."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

bf16 = torch.bfloat16


def _rand(*shape, scale=1.0):
  return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(bf16)


def _rel_err(a, b):
  a, b = a.float(), b.float()
  return ((a - b).norm() / (b.norm() + 1e-12)).item()


SHAPES = [
    (1, 512, 256),
    (8, 4096, 4096),
    (16, 6144, 4096),
    (24, 1000, 1104),       # ragged slab and k-block tails
    (64, 6144, 4096),       # Qwen3-8B fused qkv
    (64, 4096, 12288),      # down projection: 192 k-blocks per slab
    (100, 264, 200),
    (128, 4096, 4096),
    (48, 19000, 512),       # more slabs than SMs
]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_skinny_matches_fp32(kernel_lib, M, N, K):
  from tunix_b200.ops import _lib, kernels
  torch.manual_seed(M + N)
  x, w = _rand(M, K, scale=0.5), _rand(N, K, scale=0.5)
  ref = x.float() @ w.float().t()
  for _ in range(3):          # the scratch is left zeroed: repeats must agree
    out = kernels.gemm_skinny(x, w)
    _lib.check_status()
    assert _rel_err(out, ref) < 6e-3, _rel_err(out, ref)
  torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2 * math.sqrt(K) * 0.25)


@pytest.mark.parametrize("kind", ["silu", "gelu"])
@pytest.mark.parametrize("M,F,K", [(16, 1024, 512), (64, 12288, 4096), (128, 2048, 1024), (40, 1000, 264)])
def test_skinny_gated(kernel_lib, kind, M, F, K):
  from tunix_b200.ops import _lib, kernels
  torch.manual_seed(F)
  x, w = _rand(M, K, scale=0.5), _rand(2 * F, K, scale=0.1)
  gu = x.float() @ w.float().t()
  g, u = gu[:, :F], gu[:, F:]
  act = torch.nn.functional.silu(g) if kind == "silu" else torch.nn.functional.gelu(g, approximate="tanh")
  ref = act * u
  for _ in range(2):
    out = kernels.gemm_skinny(x, w, glu=kind)
    _lib.check_status()
    assert out.shape == (M, F)
    assert _rel_err(out, ref) < 8e-3, _rel_err(out, ref)


def test_skinny_residual_and_bias_in_place(kernel_lib):
  from tunix_b200.ops import _lib, kernels
  torch.manual_seed(3)
  M, N, K = 64, 4096, 4096
  x, w, h, b = _rand(M, K, scale=0.5), _rand(N, K, scale=0.05), _rand(M, N), _rand(N)
  ref = h.float() + b.float() + x.float() @ w.float().t()
  out = h.clone()
  kernels.gemm_skinny(x, w, out=out, residual=out, bias=b)
  _lib.check_status()
  assert _rel_err(out, ref) < 6e-3


def test_skinny_deterministic_mode_is_bitwise_repeatable(kernel_lib):
  from tunix_b200.ops import _lib, kernels
  torch.manual_seed(5)
  x, w = _rand(64, 4096), _rand(4096, 4096, scale=0.05)
  _lib.set_deterministic(True)
  try:
    a = kernels.gemm_skinny(x, w)
    b = kernels.gemm_skinny(x, w)
    big = kernels.gemm(x, w)        # the training-path kernel: one pass over K in the same block order
  finally:
    _lib.set_deterministic(False)
  _lib.check_status()
  assert torch.equal(a, b)
  assert _rel_err(a, big) < 1e-3


def test_linear_routes_decode_shapes_to_skinny(kernel_lib):
  from tunix_b200.ops import _lib, functional as F
  torch.manual_seed(9)
  x, w = _rand(2, 32, 1024), _rand(3072, 1024, scale=0.05)
  before = _lib.launch_calls
  with torch.no_grad():
    y = F.linear(x, w)
  assert _lib.launch_calls == before + 1           # one launch: no memset, no conversion pass
  assert _rel_err(y.reshape(64, -1), x.reshape(64, -1).float() @ w.float().t()) < 6e-3
