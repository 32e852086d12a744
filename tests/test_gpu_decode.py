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
