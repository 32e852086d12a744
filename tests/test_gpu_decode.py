"""Rollout kernels (KV page write, paged decode attention, sampling) against PyTorch references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def make_cache(B, lens, page, Kh, H, dev, extra_pages=3):
  blocks = [(n + page - 1) // page for n in lens]
  P = sum(blocks) + extra_pages
  perm = torch.randperm(P, device=dev)
  bt = torch.zeros(B, max(blocks) + 1, dtype=torch.int32, device=dev)
  off = 0
  for b, nb in enumerate(blocks):
    bt[b, :nb] = perm[off:off + nb].int()
    off += nb
  kp = torch.randn(P, page, Kh, H, device=dev).bfloat16()
  vp = torch.randn(P, page, Kh, H, device=dev).bfloat16()
  return kp, vp, bt, torch.tensor(lens, dtype=torch.int32, device=dev)


@pytest.mark.parametrize("H,N,Kh,page", [(128, 32, 8, 16), (128, 8, 8, 32), (64, 14, 2, 16), (256, 8, 4, 16),
                                         (128, 40, 8, 16)])
@pytest.mark.parametrize("splits", [1, 4])
def test_paged_decode_attention(kernel_lib, H, N, Kh, page, splits):
  from tunix_b200.ops import paged
  torch.manual_seed(0)
  lens = [1, 17, 300, 1025, 64]
  kp, vp, bt, sl = make_cache(len(lens), lens, page, Kh, H, "cuda")
  q = torch.randn(len(lens), N, H, device="cuda").bfloat16()
  scale = 1 / math.sqrt(H)
  out = paged.paged_decode_attention(q, kp, vp, bt, sl, scale, num_splits=splits)
  ref = paged.paged_decode_attention_ref(q, kp, vp, bt, sl, scale)
  torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("N,Kh,page", [(32, 8, 8), (32, 8, 64), (32, 2, 16), (4, 4, 32)])
@pytest.mark.parametrize("splits", [1, 3])
def test_paged_decode_tensor_core_kernel(kernel_lib, N, Kh, page, splits):
  """tcgen05 kernel: page sizes 8..64, groups up to 16 heads, unused block-table entries poisoned."""
  from tunix_b200.ops import _lib, paged
  torch.manual_seed(4)
  H = 128
  assert paged.tc_supported(H, page, N // Kh)
  lens = [1, 63, 64, 65, 700, 129, 2048]
  kp, vp, bt, sl = make_cache(len(lens), lens, page, Kh, H, "cuda")
  for b, n in enumerate(lens):
    bt[b, (n + page - 1) // page:] = -1          # entries past the sequence must never be dereferenced
  q = torch.randn(len(lens), N, H, device="cuda").bfloat16()
  scale = 1 / math.sqrt(H)
  out = paged.paged_decode_attention(q, kp, vp, bt, sl, scale, num_splits=splits)
  _lib.check_status()
  bt_ref = bt.clamp(min=0)
  ref = paged.paged_decode_attention_ref(q, kp, vp, bt_ref, sl, scale)
  torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_paged_decode_simt_kernel_still_matches(kernel_lib, monkeypatch):
  from tunix_b200.ops import paged
  monkeypatch.setenv("TUNIX_B200_DECODE_TC", "0")
  torch.manual_seed(5)
  H, N, Kh, page = 128, 32, 8, 16
  assert not paged.tc_supported(H, page, N // Kh)
  lens = [5, 400, 1025]
  kp, vp, bt, sl = make_cache(len(lens), lens, page, Kh, H, "cuda")
  q = torch.randn(len(lens), N, H, device="cuda").bfloat16()
  for splits in (1, 4):
    out = paged.paged_decode_attention(q, kp, vp, bt, sl, 1 / math.sqrt(H), num_splits=splits)
    ref = paged.paged_decode_attention_ref(q, kp, vp, bt, sl, 1 / math.sqrt(H))
    torch.testing.assert_close(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_kv_page_write(kernel_lib):
  from tunix_b200.ops import paged
  torch.manual_seed(1)
  P, page, Kh, H, T = 20, 16, 4, 128, 50
  kp = torch.zeros(P, page, Kh, H, device="cuda", dtype=torch.bfloat16)
  vp = torch.zeros_like(kp)
  kp2, vp2 = kp.clone(), vp.clone()
  qkv = torch.randn(T, (8 + 2 * Kh) * H, device="cuda").bfloat16()
  k = qkv[:, 8 * H:(8 + Kh) * H].view(T, Kh, H)
  v = qkv[:, (8 + Kh) * H:].view(T, Kh, H)
  slots = torch.randperm(P * page, device="cuda")[:T]
  slots[3] = -1
  paged.kv_page_write(k, v, slots, kp, vp)
  paged.kv_page_write_ref(k, v, slots, kp2, vp2)
  assert torch.equal(kp, kp2) and torch.equal(vp, vp2)


def test_sampling_greedy_and_logprob(kernel_lib):
  from tunix_b200.ops import paged
  torch.manual_seed(2)
  for dt in (torch.float32, torch.bfloat16):
    logits = (torch.randn(9, 151936, device="cuda") * 3).to(dt)
    forb = torch.tensor([5, int(logits[0].float().argmax())], dtype=torch.int32, device="cuda")
    tok, lp = paged.sample(logits, greedy=True, forbidden=forb)
    rt, rlp = paged.sample_ref(logits, 1.0, True, None, forb.tolist())
    assert torch.equal(tok, rt)
    torch.testing.assert_close(lp, rlp, rtol=1e-4, atol=1e-4)


def test_sampling_distribution_and_reproducibility(kernel_lib):
  from tunix_b200.ops import paged
  torch.manual_seed(3)
  V, B = 50, 4096
  row = torch.randn(V, device="cuda") * 1.5
  logits = row[None].expand(B, V).contiguous()
  T = 0.7
  counts = torch.zeros(V, device="cuda")
  for step in range(8):
    tok, lp = paged.sample(logits, temperature=T, seed=11, step=step)
    counts += torch.bincount(tok, minlength=V).float()
    torch.testing.assert_close(lp, torch.log_softmax(row / T, -1)[tok], rtol=1e-4, atol=1e-4)
  p = torch.softmax(row / T, -1)
  n = counts.sum()
  # every cell within 5 sigma of the binomial expectation
  assert ((counts - n * p).abs() <= 5 * torch.sqrt(n * p * (1 - p)) + 2).all()
  a, _ = paged.sample(logits, temperature=T, seed=11, step=3)
  b, _ = paged.sample(logits, temperature=T, seed=11, step=3)
  st = torch.tensor(2, dtype=torch.int64, device="cuda")
  c, _ = paged.sample(logits, temperature=T, seed=11, step=1, step_tensor=st)
  d, _ = paged.sample(logits, temperature=T, seed=12, step=3)
  assert torch.equal(a, b) and torch.equal(a, c) and not torch.equal(a, d)
  # rows draw independently
  assert len(torch.unique(a)) > 5


def _survivors_ref(z, top_k, top_p):
  """Boolean [V] mask of the tokens the reference rule keeps (sorted cumsum over the top-k candidates)."""
  V = z.numel()
  k = V if not top_k or top_k <= 0 else min(top_k, V)
  zs, idx = torch.topk(z, k)
  keep = torch.ones(k, dtype=torch.bool, device=z.device)
  if top_p is not None and top_p < 1.0:
    ps = torch.softmax(zs, -1)
    keep = ~(torch.cumsum(ps, -1) - ps > top_p)
  mask = torch.zeros(V, dtype=torch.bool, device=z.device)
  mask[idx[keep]] = True
  return mask


@pytest.mark.parametrize("top_k,top_p", [(5, None), (None, 0.6), (40, 0.9), (1, None), (None, 0.999)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_sampling_top_k_top_p_in_kernel(kernel_lib, top_k, top_p, dtype):
  """Draws stay inside the reference's survivor set, follow its renormalised distribution, report the
  log-prob under the full distribution, and repeat bit for bit."""
  from tunix_b200.ops import paged
  torch.manual_seed(4)
  V, B, T = 2000, 4096, 0.8
  row = (torch.randn(V, device="cuda") * 2.5).to(dtype)
  logits = row[None].expand(B, V).contiguous()
  z = row.float() / T
  keep = _survivors_ref(z, top_k, top_p)
  counts = torch.zeros(V, device="cuda")
  for step in range(4):
    tok, lp = paged.sample(logits, temperature=T, seed=3, step=step, top_k=top_k, top_p=top_p)
    assert keep[tok].all(), "a token outside the top-k / top-p set was drawn"
    counts += torch.bincount(tok, minlength=V).float()
    torch.testing.assert_close(lp, torch.log_softmax(z, -1)[tok], rtol=1e-4, atol=2e-4)
  p = torch.softmax(torch.where(keep, z, torch.full_like(z, float("-inf"))), -1)
  n = counts.sum()
  # the kernel may keep ties of the boundary bin: allow the boundary token(s) to differ, test the rest
  assert ((counts - n * p).abs() <= 5 * torch.sqrt(n * p * (1 - p)) + 3).float().mean() > 0.999
  a, _ = paged.sample(logits, temperature=T, seed=3, step=1, top_k=top_k, top_p=top_p)
  b, _ = paged.sample(logits, temperature=T, seed=3, step=1, top_k=top_k, top_p=top_p)
  assert torch.equal(a, b)


def test_sampling_filtered_large_vocab_and_forbidden(kernel_lib):
  from tunix_b200.ops import paged
  torch.manual_seed(6)
  logits = (torch.randn(16, 151936, device="cuda") * 3).bfloat16()
  best = logits.float().argmax(-1)
  forb = torch.tensor([int(best[0])], dtype=torch.int32, device="cuda")
  tok, lp = paged.sample(logits, temperature=1.0, seed=1, top_k=1, forbidden=forb)
  z = logits.float().clone()
  z[:, int(best[0])] = float("-inf")
  # top-1 sampling draws a maximum of what is allowed (bf16 rows have exact ties at the top: any of them)
  assert torch.equal(z.gather(-1, tok[:, None])[:, 0], z.max(-1).values)
  assert int(tok[0]) != int(best[0])
  torch.testing.assert_close(lp, torch.log_softmax(z, -1).gather(-1, tok[:, None])[:, 0], rtol=1e-4, atol=2e-4)


def test_qknorm_rope_writes_pages_in_the_same_launch(kernel_lib):
  from tunix_b200.ops import kernels, paged
  torch.manual_seed(8)
  T, NQ, NK, H, page, P = 24, 8, 2, 128, 16, 10
  x = torch.randn(T, (NQ + 2 * NK) * H, device="cuda").bfloat16()
  pos = torch.randint(0, 500, (T,), device="cuda", dtype=torch.int32)
  wq, wk = torch.randn(H, device="cuda").bfloat16(), torch.randn(H, device="cuda").bfloat16()
  table = kernels.rope_table(512, H, 10000.0, "cuda")
  slots = torch.randperm(P * page, device="cuda")[:T].long()
  slots[3] = -1
  kp = torch.zeros(P, page, NK, H, device="cuda").bfloat16()
  vp = torch.zeros_like(kp)
  fused = kernels.qknorm_rope_fwd(x, pos, table, NQ, NK, H, wq, wk, 1e-6, slots=slots, k_pages=kp, v_pages=vp)
  plain = kernels.qknorm_rope_fwd(x, pos, table, NQ, NK, H, wq, wk, 1e-6)
  assert torch.equal(fused, plain)
  kp2, vp2 = torch.zeros_like(kp), torch.zeros_like(vp)
  k = plain[:, NQ * H:(NQ + NK) * H].reshape(T, NK, H)
  v = plain[:, (NQ + NK) * H:].reshape(T, NK, H)
  paged.kv_page_write_ref(k, v, slots, kp2, vp2)
  assert torch.equal(kp, kp2) and torch.equal(vp, vp2)


def test_rope_position_beyond_the_table_is_reported_not_read(kernel_lib):
  from tunix_b200.ops import _lib, kernels
  H = 128
  x = torch.randn(4, 3 * H, device="cuda").bfloat16()
  table = kernels.rope_table(64, H, 10000.0, "cuda")
  rows = table.shape[0]
  _lib.check_status()
  ok = kernels.qknorm_rope_fwd(x, torch.tensor([0, 1, 2, rows - 1], device="cuda", dtype=torch.int32), table, 1, 1, H)
  _lib.check_status()
  bad = kernels.qknorm_rope_fwd(x, torch.tensor([0, 1, 2, rows + 5], device="cuda", dtype=torch.int32), table, 1, 1, H)
  with pytest.raises(RuntimeError, match="0x8"):
    _lib.check_status()
  assert torch.equal(ok, bad)         # clamped to the last row, nothing read out of range
  _lib.check_status()                 # the word was cleared: the context is still usable
