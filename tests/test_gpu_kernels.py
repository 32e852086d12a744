"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

bf16 = torch.bfloat16


def _rand(*shape, scale=1.0, dtype=bf16):
  return (torch.randn(*shape, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _rel_err(a, b):
  a = a.float()
  b = b.float()
  return ((a - b).norm() / (b.norm() + 1e-12)).item()


GEMM_SHAPES = [
    (128, 256, 64),
    (256, 512, 512),
    (384, 1024, 4096),
    (1000, 264, 200),     # ragged in every dimension (multiples of 8)
    (4096, 6144, 4096),   # Llama-8B fused qkv
    (8, 128, 128),
    (2048, 1024, 4096),
    (2304, 4608, 512),    # CTA-pair kernel, exact tiles
    (2200, 4360, 264),    # CTA-pair kernel, ragged in M, N and K
    (8192, 4096, 1024),
    (64, 512, 4096),      # skinny: 64-column tiles, K split 8 ways, fp32 atomics + rounding pass
    (40, 264, 1104),      # skinny and ragged, K split 2 ways
    (128, 4096, 12288),   # decode down-projection
]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True), (True, False)])
def test_gemm_layouts(kernel_lib, M, N, K, a_mn, b_mn):
  from tunix_b200.ops import _lib, kernels
  torch.manual_seed(0)
  a = _rand(M, K, scale=0.5)
  b = _rand(N, K, scale=0.5)
  ref = a.float() @ b.float().t()
  a_in = a.t().contiguous() if a_mn else a
  b_in = b.t().contiguous() if b_mn else b
  out = kernels.gemm(a_in, b_in, a_mn=a_mn, b_mn=b_mn)
  _lib.check_status()
  assert out.shape == (M, N)
  assert _rel_err(out, ref) < 6e-3, _rel_err(out, ref)
  # elementwise check too (bf16 output rounding dominates)
  torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2 * math.sqrt(K) * 0.25)


def test_skinny_gemm_scratch_is_left_clean(kernel_lib):
  """Decode-shaped GEMMs share one zero-filled scratch: interleaved shapes and repeats must not leak."""
  from tunix_b200.ops import _lib, kernels
  torch.manual_seed(7)
  shapes = [(64, 4096, 4096), (100, 1024, 2048), (8, 6144, 4096), (128, 4096, 12288), (64, 4096, 4096), (1, 512, 1024)]
  for rep in range(2):
    for M, N, K in shapes:
      a, b = _rand(M, K, scale=0.5), _rand(N, K, scale=0.5)
      out = kernels.gemm(a, b)
      ref = a.float() @ b.float().t()
      assert _rel_err(out, ref) < 6e-3, (M, N, K, rep, _rel_err(out, ref))
  _lib.check_status()


def test_gemm_fp32_accumulate(kernel_lib):
  from tunix_b200.ops import _lib, kernels
  torch.manual_seed(1)
  M, N, K = 512, 768, 1024
  a, b = _rand(M, K, scale=0.3), _rand(N, K, scale=0.3)
  c0 = torch.randn(M, N, device="cuda")
  out = c0.clone()
  kernels.gemm(a, b, out=out, accumulate=True, alpha=0.5)
  _lib.check_status()
  ref = c0 + 0.5 * (a.float() @ b.float().t())
  torch.testing.assert_close(out, ref, rtol=1e-3, atol=1e-2)
  # bf16 accumulate (residual add in the epilogue)
  r0 = _rand(M, N)
  out2 = r0.clone()
  kernels.gemm(a, b, out=out2, accumulate=True)
  ref2 = r0.float() + a.float() @ b.float().t()
  assert _rel_err(out2, ref2) < 6e-3


def test_gemm_strided_views(kernel_lib):
  """Operands that are column slices of wider buffers (row stride != width)."""
  from tunix_b200.ops import _lib, kernels
  torch.manual_seed(2)
  big = _rand(512, 1024, scale=0.5)
  a = big[:, 256:768]            # [512, 512], stride 1024
  w = _rand(256, 512, scale=0.5)
  out_big = torch.zeros(512, 1024, device="cuda", dtype=bf16)
  kernels.gemm(a, w, out=out_big[:, 128:384])
  _lib.check_status()
  ref = a.float() @ w.float().t()
  assert _rel_err(out_big[:, 128:384], ref) < 6e-3
  assert out_big[:, :128].abs().max().item() == 0 and out_big[:, 384:].abs().max().item() == 0


def test_gemm_pair_matches_single_cta(kernel_lib):
  """The 2-CTA kernel and the 1-CTA kernel accumulate in the same order: identical results."""
  from tunix_b200.ops import _lib, kernels
  lib = _lib.require()
  a, b = _rand(4096, 2048, scale=0.5), _rand(4608, 2048, scale=0.5)
  o_pair = kernels.gemm(a, b)
  lib.tx_gemm_set_disable_pair(1)
  try:
    o_single = kernels.gemm(a, b)
  finally:
    lib.tx_gemm_set_disable_pair(0)
  _lib.check_status()
  assert torch.equal(o_pair, o_single)


def test_gemm_deterministic(kernel_lib):
  from tunix_b200.ops import kernels
  a, b = _rand(1024, 2048), _rand(1536, 2048)
  o1 = kernels.gemm(a, b)
  o2 = kernels.gemm(a, b)
  assert torch.equal(o1, o2)


@pytest.mark.parametrize("T,D", [(37, 256), (4096, 4096), (513, 2560), (64, 8192)])
@pytest.mark.parametrize("offset", [0.0, 1.0])
def test_rmsnorm(kernel_lib, T, D, offset):
  from tunix_b200.ops import kernels
  torch.manual_seed(0)
  x, w, res, dy, dres = _rand(T, D), _rand(D, scale=0.3), _rand(T, D), _rand(T, D), _rand(T, D)
  eps = 1e-5

  def ref_fn(xf, wf):
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (wf + offset)

  y, s, rstd = kernels.rmsnorm_fwd(x, w, eps, offset)
  assert s is None
  torch.testing.assert_close(y.float(), ref_fn(x.float(), w.float()), rtol=2e-2, atol=2e-2)
  y2, s2, _ = kernels.rmsnorm_fwd(x, w, eps, offset, residual=res)
  sref = (x.float() + res.float()).to(bf16)
  assert torch.equal(s2, sref)
  torch.testing.assert_close(y2.float(), ref_fn(sref.float(), w.float()), rtol=2e-2, atol=2e-2)

  xf = x.float().requires_grad_(True)
  wf = w.float().requires_grad_(True)
  ref_fn(xf, wf).backward(dy.float())
  dx, dw = kernels.rmsnorm_bwd(x, w, dy, rstd, eps, offset, dres=dres)
  assert _rel_err(dx, xf.grad + dres.float()) < 1e-2
  assert _rel_err(dw, wf.grad) < 1e-3
  dx_b, _ = kernels.rmsnorm_bwd(x, w, dy, None, eps, offset)
  assert _rel_err(dx_b, xf.grad) < 1e-2


def _rope_ref(x, pos, theta, H):
  half = H // 2
  inv = 1.0 / (theta ** (torch.arange(half, device=x.device, dtype=torch.float32) * 2.0 / H))
  ang = pos.float()[:, None] * inv[None, :]
  cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
  x1, x2 = x[..., :half], x[..., half:]
  return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


@pytest.mark.parametrize("H", [64, 128, 256])
@pytest.mark.parametrize("qk_norm", [False, True])
def test_qknorm_rope(kernel_lib, H, qk_norm):
  from tunix_b200.ops import kernels
  torch.manual_seed(0)
  T, NQ, NK = 300, 8, 2
  theta, eps = 1e6, 1e-6
  x = _rand(T, (NQ + 2 * NK) * H)
  pos = torch.randint(0, 2048, (T,), device="cuda", dtype=torch.int32)
  table = kernels.rope_table(2048, H, theta, "cuda")
  wq = _rand(H, scale=0.5) if qk_norm else None
  wk = _rand(H, scale=0.5) if qk_norm else None

  def ref_fn(xf, wqf, wkf):
    xh = xf.view(T, NQ + 2 * NK, H)
    q, k, v = xh[:, :NQ], xh[:, NQ:NQ + NK], xh[:, NQ + NK:]
    if qk_norm:
      q = q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + eps) * wqf
      k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + eps) * wkf
    return torch.cat([_rope_ref(q, pos, theta, H), _rope_ref(k, pos, theta, H), v], dim=1).reshape(T, -1)

  out = kernels.qknorm_rope_fwd(x, pos, table, NQ, NK, H, wq, wk, eps)
  xf = x.float().requires_grad_(True)
  wqf = wq.float().requires_grad_(True) if qk_norm else None
  wkf = wk.float().requires_grad_(True) if qk_norm else None
  ref = ref_fn(xf, wqf, wkf)
  assert _rel_err(out, ref) < 1e-2
  dy = _rand(T, (NQ + 2 * NK) * H)
  ref.backward(dy.float())
  dx, dwq, dwk = kernels.qknorm_rope_bwd(x, dy, pos, table, NQ, NK, H, wq, wk, eps)
  assert _rel_err(dx, xf.grad) < 1e-2
  if qk_norm:
    assert _rel_err(dwq, wqf.grad) < 1e-2
    assert _rel_err(dwk, wkf.grad) < 1e-2


@pytest.mark.parametrize("gelu", [False, True])
def test_glu(kernel_lib, gelu):
  from tunix_b200.ops import kernels
  torch.manual_seed(0)
  T, F = 777, 1536
  gu, dout = _rand(T, 2 * F), _rand(T, F)
  guf = gu.float().requires_grad_(True)
  g, u = guf[:, :F], guf[:, F:]
  act = torch.nn.functional.gelu(g, approximate="tanh") if gelu else torch.nn.functional.silu(g)
  ref = act * u
  out = kernels.glu_fwd(gu, gelu)
  assert _rel_err(out, ref) < 1e-2
  ref.backward(dout.float())
  dgu = kernels.glu_bwd(gu, dout, gelu)
  assert _rel_err(dgu, guf.grad) < 1e-2


def test_embedding(kernel_lib):
  from tunix_b200.ops import kernels
  torch.manual_seed(0)
  V, D, T = 1000, 512, 4096
  table = _rand(V, D)
  ids = torch.randint(0, V, (T,), device="cuda")
  out = kernels.embedding_fwd(ids, table, scale=2.0)
  assert _rel_err(out, table.float()[ids] * 2.0) < 5e-3
  dout = _rand(T, D)
  grad = torch.zeros(V, D, device="cuda")
  kernels.embedding_bwd(ids, dout, grad, scale=2.0)
  ref = torch.zeros(V, D, device="cuda").index_add_(0, ids, dout.float() * 2.0)
  torch.testing.assert_close(grad, ref, rtol=1e-4, atol=1e-3)


def test_adamw_and_norm(kernel_lib):
  from tunix_b200.ops import kernels
  torch.manual_seed(0)
  n = 1_000_003
  p0 = torch.randn(n, device="cuda")
  g = torch.randn(n, device="cuda")
  master, m, v = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
  pb = torch.empty(n, device="cuda", dtype=bf16)
  ref_p = torch.nn.Parameter(p0.clone())
  opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
  # gradient norm + clip factor on device
  ss = torch.zeros(1, device="cuda")
  kernels.sumsq(g, ss)
  torch.testing.assert_close(ss[0], g.double().pow(2).sum().float(), rtol=1e-5, atol=0)
  inv_denom = torch.full((1,), 0.25, device="cuda")
  norm, scale = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
  kernels.clip_scale(ss, inv_denom, 1.0, norm, scale)
  gn = (g * 0.25).norm()
  torch.testing.assert_close(norm[0], gn, rtol=1e-5, atol=0)
  torch.testing.assert_close(scale[0], 0.25 / (gn + 1e-6), rtol=1e-5, atol=0)
  for step in range(1, 4):
    gi = g * step
    ref_p.grad = (gi * scale).clone()
    opt.step()
    grad_buf = gi.clone()
    kernels.adamw_step(master, m, v, grad_buf, pb, lr=1e-2, beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                       step=step, grad_scale=scale, zero_grad=True)
    assert grad_buf.abs().max().item() == 0
  torch.testing.assert_close(master, ref_p.data, rtol=1e-4, atol=1e-5)
  assert torch.equal(pb, master.to(bf16))


@pytest.mark.parametrize("dtype", [torch.float32, bf16])
@pytest.mark.parametrize("softcap", [0.0, 30.0])
def test_logprob(kernel_lib, dtype, softcap):
  from tunix_b200.ops import kernels
  torch.manual_seed(0)
  T, V, Vp = 257, 5003, 5008
  logits = _rand(T, Vp, scale=3.0, dtype=dtype)
  tgt = torch.randint(0, V, (T,), device="cuda")
  inv_temp = 1.0 / 0.7
  lf = logits[:, :V].float().requires_grad_(True)
  z = lf
  if softcap > 0:
    z = softcap * torch.tanh(z / softcap)
  z = z * inv_temp
  lsm = torch.log_softmax(z, dim=-1)
  ref_lp = lsm.gather(1, tgt[:, None])[:, 0]
  ref_ent = -(lsm.exp() * lsm).sum(-1)
  lp, lse, ent = kernels.logprob_fwd(logits, tgt, inv_temp, softcap, want_entropy=True, n_valid=V)
  torch.testing.assert_close(lp, ref_lp, rtol=1e-4, atol=1e-4)
  torch.testing.assert_close(ent, ref_ent, rtol=1e-3, atol=1e-3)
  g_lp = torch.randn(T, device="cuda")
  g_ent = torch.randn(T, device="cuda") * 0.1
  (ref_lp * g_lp + ref_ent * g_ent).sum().backward()
  dl = kernels.logprob_bwd(logits, tgt, lse, ent, g_lp, g_ent, inv_temp, softcap, n_valid=V)
  assert dl.shape == (T, Vp)
  assert dl[:, V:].abs().max().item() == 0
  assert _rel_err(dl[:, :V], lf.grad) < 1e-2


@pytest.mark.parametrize("multi", [False, True])
def test_fused_lora_linear_matches_unfused(kernel_lib, multi):
  """Adapters folded into the base GEMM as extra K blocks: forward, dx, dA and dB against the three-GEMM form."""
  from tunix_b200.models.transformer import Linear
  from tunix_b200.ops import _lib, lora as lora_ops
  torch.manual_seed(11)
  T, din, dout = 384, 512, 1536
  slices = {"q_proj": (0, 1024), "k_proj": (1024, 1280), "v_proj": (1280, 1536)} if multi else None
  lin = Linear(din, dout, False, torch.bfloat16, "cuda", slices)
  with torch.no_grad():
    lin.w.normal_(0, 0.05)
  lin.w.requires_grad_(False)
  for name, rank in ((("q_proj", 16), ("k_proj", 8), ("v_proj", 8)) if multi else (("", 16),)):
    lin.add_lora(name, rank, 32.0)
  with torch.no_grad():
    for b in lin.lora_b.values():
      b.normal_(0, 0.05)
  x = (torch.randn(2, T // 2, din, device="cuda") * 0.5).bfloat16().requires_grad_()
  assert lora_ops.supported(x.reshape(-1, din), lin.w, lin._adapters())
  y = lin(x)
  dy = torch.randn_like(y)
  y.backward(dy)
  _lib.check_status()
  got = [y.detach().float(), x.grad.float()] + [p.grad.float() for p in list(lin.lora_a.values()) + list(lin.lora_b.values())]
  # fp32 restatement
  xr = x.detach().float().requires_grad_()
  As = [a.detach().float().requires_grad_() for a in lin.lora_a.values()]
  Bs = [b.detach().float().requires_grad_() for b in lin.lora_b.values()]
  yr = xr @ lin.w.float().t()
  parts = []
  for (key, _), a, b in zip(lin.lora_a.items(), As, Bs):
    lo, hi = lin.slices["" if key == "w" else key]
    d = (xr @ a.t()) @ b.t() * lin.lora_scale[key]
    parts.append((lo, hi, d))
  yr = yr + torch.cat([d for _, _, d in sorted(parts)], dim=-1) if multi else yr + parts[0][2]
  yr.backward(dy.float())
  want = [yr.detach(), xr.grad] + [a.grad for a in As] + [b.grad for b in Bs]
  for i, (g, w) in enumerate(zip(got, want)):
    err = (g - w).norm() / (w.norm() + 1e-6)
    assert err < 2e-2, (i, err.item())


@pytest.mark.parametrize("world,rank,slab", [(1, 0, 128), (2, 0, 128), (2, 1, 256), (4, 2, 128), (4, 3, 256)])
def test_gemm_with_fused_allgather_of_sharded_weight(kernel_lib, world, rank, slab):
  """The all-gather-into-GEMM kernel with every "rank's" shard on this one GPU (a single launch: the copy warps
  and the tensor-core warps of the same kernel hand slabs over through counters)."""
  from tunix_b200.ops import _lib, kernels
  torch.manual_seed(11)
  M, K, N = 384, 256, (128 * world * 3 if slab == 128 else 256 * world * 2)   # the kernel picks 256-row slabs when it can
  a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
  w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) / K ** 0.5
  shards = [w[r * (N // world):(r + 1) * (N // world)].clone() for r in range(world)]
  stage = torch.full((N, K), float("nan"), device="cuda", dtype=torch.bfloat16)
  cnt = torch.empty(N // 128, device="cuda", dtype=torch.int32)
  for _ in range(2):                                   # a second call reuses the scratch
    c = kernels.gemm_allgather_b(a, [s.data_ptr() for s in shards], rank, N // world, stage, cnt)
  torch.cuda.synchronize()
  _lib.check_status(torch.device("cuda"))
  ref = a.float() @ w.float().t()
  assert torch.allclose(c.float(), ref, atol=3e-2, rtol=3e-2)
  # the staging buffer holds exactly the remote shards; the local rows were read in place
  per = N // world
  for r in range(world):
    blk = stage[r * per:(r + 1) * per]
    if r == rank:
      assert bool(torch.isnan(blk.float()).all())
    else:
      assert torch.equal(blk, shards[r])
  assert int(cnt.min()) == int(cnt.max()) or world > 1


def test_deterministic_mode_makes_skinny_gemms_bitwise_reproducible(kernel_lib):
  from tunix_b200.ops import _lib, kernels
  torch.manual_seed(12)
  a = torch.randn(64, 12288, device="cuda", dtype=torch.bfloat16)
  w = torch.randn(4096, 12288, device="cuda", dtype=torch.bfloat16) / 110.0
  ref = a.float() @ w.float().t()
  _lib.set_deterministic(True)
  try:
    outs = [kernels.gemm(a, w).clone() for _ in range(4)]
  finally:
    _lib.set_deterministic(False)
  assert all(torch.equal(outs[0], o) for o in outs[1:])
  assert torch.allclose(outs[0].float(), ref, atol=5e-2, rtol=3e-2)
  assert torch.allclose(kernels.gemm(a, w).float(), ref, atol=5e-2, rtol=3e-2)       # split-K path back on


def test_debug_build_reports_indices_the_release_build_clamps(kernel_lib):
  """The -DTX_DEBUG library records an out-of-range token id (the release kernel clamps it silently)."""
  import os
  import subprocess
  import sys
  from tunix_b200 import build_kernels
  build_kernels.build(debug=True)
  code = r"""
import torch
from tunix_b200.ops import _lib, kernels
table = torch.randn(16, 64, device="cuda").bfloat16()
ok = kernels.embedding_fwd(torch.tensor([0, 15, 3], device="cuda", dtype=torch.int32), table)
_lib.status_word("cuda"); _lib.check_status()
bad = kernels.embedding_fwd(torch.tensor([0, 99, 3], device="cuda", dtype=torch.int32), table)
assert torch.equal(bad[1], table[15])            # still clamped: no fault
try:
  _lib.check_status()
  print("NO_REPORT")
except RuntimeError as e:
  print("REPORT", e)
_lib.check_status()                               # the record was cleared
print("DONE")
"""
  root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
  for debug, want in (("1", "REPORT"), ("0", "NO_REPORT")):
    r = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, TUNIX_B200_DEBUG_KERNELS=debug, PYTHONPATH=root),
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert want in r.stdout and "DONE" in r.stdout, r.stdout
    if debug == "1":
      assert "token id outside the vocabulary" in r.stdout and "value 99, limit 16" in r.stdout
