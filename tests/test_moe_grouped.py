"""Grouped expert MLP: the device-side padded layout (CPU) and the grouped tcgen05 GEMM (GPU)."""
import pytest
import torch

from tunix_b200.ops import moe as moe_ops


def test_padded_layout_places_every_row_in_its_experts_block():
  torch.manual_seed(0)
  E, n = 5, 700
  ids = torch.randint(0, E, (n,))
  ids[ids == 3] = 1                       # expert 3 gets no rows
  lay = moe_ops.padded_layout(ids, E)
  assert lay.rows == moe_ops.padded_rows(n, E) and lay.rows % 128 == 0
  off = lay.offsets.tolist()
  assert all(o % 128 == 0 for o in off) and off[3] == off[4]
  assert lay.dest.unique().numel() == n                        # no two rows share a slot
  for i in range(n):
    e = int(ids[i])
    assert off[e] <= int(lay.dest[i]) < off[e] + int((ids == e).sum())
  # rows of one expert keep their original order
  d1 = lay.dest[ids == 1]
  assert torch.all(d1[1:] > d1[:-1])
  te = lay.tile_expert.tolist()
  for t, e in enumerate(te):
    if t * 128 < off[E]:
      assert off[e] <= t * 128 < off[e + 1]
    else:
      assert e == -1


def _ref_grouped(x_pad, w, lay):
  y = torch.zeros(lay.rows, w.shape[1], dtype=torch.float32, device=x_pad.device)
  off = lay.offsets.tolist()
  for e in range(lay.num_experts):
    y[off[e]:off[e + 1]] = x_pad[off[e]:off[e + 1]].float() @ w[e].float().t()
  return y


@pytest.mark.gpu
@pytest.mark.parametrize("E,N,K,n", [(8, 256, 128, 1500), (16, 1536, 2048, 5000), (4, 192, 72, 300), (128, 128, 64, 2000)])
def test_grouped_gemm_forward_dgrad_wgrad(kernel_lib, E, N, K, n):
  torch.manual_seed(1)
  dev = "cuda"
  ids = torch.randint(0, E, (n,), device=dev)
  ids[ids == 2] = 0                       # an expert without rows
  lay = moe_ops.padded_layout(ids, E)
  x = torch.randn(n, K, device=dev, dtype=torch.bfloat16)
  x_pad = torch.zeros(lay.rows, K, device=dev, dtype=torch.bfloat16).index_copy(0, lay.dest, x).requires_grad_()
  w = (torch.randn(E, N, K, device=dev, dtype=torch.bfloat16) / K ** 0.5).requires_grad_()
  y = moe_ops.grouped_linear(x_pad, w, lay)
  ref = _ref_grouped(x_pad.detach(), w.detach(), lay)
  used = torch.zeros(lay.rows, dtype=torch.bool, device=dev)
  used[lay.dest] = True
  assert torch.allclose(y.float()[used], ref[used], atol=2e-2, rtol=2e-2)
  assert float(y.float()[~used].abs().max()) == 0.0          # padding rows stay zero
  dy = torch.zeros_like(y)
  dy[used] = torch.randn(int(used.sum()), N, device=dev, dtype=torch.bfloat16)
  y.backward(dy)
  xr = x_pad.detach().float().requires_grad_()
  wr = w.detach().float().requires_grad_()
  off = lay.offsets.tolist()
  yr = torch.cat([xr[off[e]:off[e + 1]] @ wr[e].t() for e in range(E)] + [xr[off[E]:] @ wr[0].t() * 0])
  yr.backward(dy.float())
  assert torch.allclose(x_pad.grad.float()[used], xr.grad[used], atol=3e-2, rtol=3e-2)
  scale = float(wr.grad.abs().max()) + 1e-6
  assert float((w.grad.float() - wr.grad).abs().max()) / scale < 2e-2
  assert float(w.grad[2].abs().max()) == 0.0
  from tunix_b200.ops import _lib
  _lib.check_status(torch.device(dev))


@pytest.mark.gpu
def test_grouped_wgrad_accumulates_into_main_grad(kernel_lib):
  torch.manual_seed(2)
  dev, E, N, K, n = "cuda", 6, 128, 256, 900
  ids = torch.randint(0, E, (n,), device=dev)
  lay = moe_ops.padded_layout(ids, E)
  x_pad = torch.zeros(lay.rows, K, device=dev, dtype=torch.bfloat16)
  x_pad[lay.dest] = torch.randn(n, K, device=dev, dtype=torch.bfloat16)
  w = torch.nn.Parameter(torch.randn(E, N, K, device=dev, dtype=torch.bfloat16) * 0.05)
  w.main_grad = torch.ones(E, N, K, device=dev, dtype=torch.float32)
  y = moe_ops.grouped_linear(x_pad, w, lay)
  dy = torch.zeros_like(y)
  dy[lay.dest] = torch.randn(n, N, device=dev, dtype=torch.bfloat16)
  y.backward(dy)
  assert w.grad is None
  off = lay.offsets.tolist()
  for e in range(E):
    ref = 1.0 + dy[off[e]:off[e + 1]].float().t() @ x_pad[off[e]:off[e + 1]].float()
    assert torch.allclose(w.main_grad[e], ref, atol=5e-2, rtol=2e-2)


@pytest.mark.gpu
def test_moe_layer_grouped_path_matches_expert_loop(kernel_lib):
  from tunix_b200.models.transformer import ModelConfig, MoELayer
  torch.manual_seed(3)
  cfg = ModelConfig(vocab_size=64, embed_dim=128, hidden_dim=64, num_layers=1, num_heads=2, num_kv_heads=1, head_dim=64,
                    num_experts=8, num_experts_per_tok=2, moe_hidden_dim=64, norm_topk_prob=True, dtype=torch.bfloat16)
  layer = MoELayer(cfg, device="cuda")
  for p in layer.parameters():
    torch.nn.init.normal_(p, std=0.08)
  x = torch.randn(2, 96, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
  assert moe_ops.grouped_supported(x.reshape(-1, 128), layer.gate_up_proj)
  y = layer(x)
  y.float().square().sum().backward()
  g_fast = [p.grad.float().clone() for p in layer.parameters()] + [x.grad.float().clone()]
  for p in layer.parameters():
    p.grad = None
  x.grad = None
  real = moe_ops.grouped_supported
  moe_ops.grouped_supported = lambda *_: False
  try:
    y2 = layer(x)
    y2.float().square().sum().backward()
  finally:
    moe_ops.grouped_supported = real
  g_ref = [p.grad.float() for p in layer.parameters()] + [x.grad.float()]
  assert torch.allclose(y.float(), y2.float(), atol=2e-2, rtol=2e-2)
  for a, b in zip(g_fast, g_ref):
    assert float((a - b).abs().max()) <= 3e-2 * (float(b.abs().max()) + 1e-3)


def test_peer_plan_emulated_ranks_reproduce_the_dense_moe():
  """The expert-parallel placement, checked on CPU by playing all ranks in one process: rows are scattered
  into per-rank buffers at the planned (rank, row), each rank runs its experts over its padded blocks, and
  tokens pull their k results back."""
  from tunix_b200.dist import moe as dist_moe
  torch.manual_seed(4)
  ep, E, k, T, D, Fh = 4, 8, 2, 50, 16, 24
  per = E // ep
  w1 = torch.randn(E, Fh, D) * 0.3
  w2 = torch.randn(E, D, Fh) * 0.3
  xs = [torch.randn(T, D) for _ in range(ep)]
  topi = [torch.stack([torch.randperm(E)[:k] for _ in range(T)]) for _ in range(ep)]
  for r in range(ep):
    topi[r][topi[r] == 5] = 4                              # expert 5 receives nothing
  topv = [torch.rand(T, k) for _ in range(ep)]
  table = torch.stack([torch.bincount(topi[r].reshape(-1), minlength=E) for r in range(ep)])
  capacity = moe_ops.padded_rows(T * k * ep, per)
  plans = [dist_moe.peer_plan(topi[r].reshape(-1), table, r, capacity) for r in range(ep)]
  recv = [torch.full((capacity, D), float("nan")) for _ in range(ep)]
  taken = [torch.zeros(capacity, dtype=torch.bool) for _ in range(ep)]
  for r in range(ep):
    p = plans[r]
    for i in range(T * k):
      d, row = int(p.dest_rank[i]), int(p.dest_row[i])
      assert d == int(topi[r].reshape(-1)[i]) // per
      assert not taken[d][row] and bool(plans[d].valid[row])
      taken[d][row] = True
      recv[d][row] = xs[r][i // k]
  send = []
  for d in range(ep):
    assert torch.equal(taken[d], plans[d].valid)             # every valid row was written exactly once
    lay = plans[d].layout
    x_rows = torch.where(plans[d].valid[:, None], recv[d], torch.zeros(()))
    off = lay.offsets.tolist()
    y = torch.zeros(capacity, D)
    for e in range(per):
      blk = x_rows[off[e]:off[e + 1]]
      y[off[e]:off[e + 1]] = torch.relu(blk @ w1[d * per + e].t()) @ w2[d * per + e].t()
      te = lay.tile_expert[off[e] // 128:off[e + 1] // 128]
      assert torch.all(te == e)
    send.append(y)
  for r in range(ep):
    p = plans[r]
    out = torch.zeros(T, D)
    for i in range(T * k):
      out[i // k] += topv[r].reshape(-1)[i] * send[int(p.dest_rank[i])][int(p.dest_row[i])]
    ref = torch.zeros(T, D)
    for t in range(T):
      for j in range(k):
        e = int(topi[r][t, j])
        ref[t] += topv[r][t, j] * (torch.relu(xs[r][t] @ w1[e].t()) @ w2[e].t())
    assert torch.allclose(out, ref, atol=1e-5)
