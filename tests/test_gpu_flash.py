"""tcgen05 flash attention forward against a plain fp32 reference."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def ref_attention(q, k, v, causal, scale):
  B, Lq, N, H = q.shape
  Lk, Kh = k.shape[1], k.shape[2]
  qf = q.float().transpose(1, 2)
  kf = k.float().transpose(1, 2).repeat_interleave(N // Kh, 1)
  vf = v.float().transpose(1, 2).repeat_interleave(N // Kh, 1)
  s = qf @ kf.transpose(-1, -2) * scale
  if causal:
    i = torch.arange(Lq, device=q.device)[:, None]
    j = torch.arange(Lk, device=q.device)[None, :]
    s = s.masked_fill(j > i + (Lk - Lq), float("-inf"))
  lse = torch.logsumexp(s, -1)
  return (torch.softmax(s, -1) @ vf).transpose(1, 2), lse


@pytest.mark.parametrize("B,Lq,Lk,N,Kh,causal", [
    (1, 128, 128, 2, 2, True), (2, 256, 256, 4, 2, True), (1, 200, 200, 4, 1, True), (2, 384, 384, 2, 2, False),
    (1, 100, 333, 2, 1, True), (1, 1024, 1024, 8, 2, True), (1, 64, 1000, 2, 2, False)])
def test_flash_fwd_matches_reference(kernel_lib, B, Lq, Lk, N, Kh, causal):
  from tunix_b200.ops import _lib, flash
  torch.manual_seed(0)
  dev = "cuda"
  H = 128
  # q, k, v as views of one fused projection output, like the decoder layer produces them
  qkv = torch.randn(B, max(Lq, Lk), (N + 2 * Kh) * H, device=dev).bfloat16()
  q = qkv[:, :Lq, :N * H].view(B, Lq, N, H) if Lq == Lk else torch.randn(B, Lq, N, H, device=dev).bfloat16()
  k = qkv[:, :Lk, N * H:(N + Kh) * H].view(B, Lk, Kh, H) if Lq == Lk else torch.randn(B, Lk, Kh, H, device=dev).bfloat16()
  v = qkv[:, :Lk, (N + Kh) * H:].view(B, Lk, Kh, H) if Lq == Lk else torch.randn(B, Lk, Kh, H, device=dev).bfloat16()
  scale = 1.0 / math.sqrt(H)
  assert flash.supported(q, k, v, None, causal)
  o, ctx = flash.forward(q, k, v, causal=causal, scale=scale)
  _lib.check_status()
  o_ref, lse_ref = ref_attention(q, k, v, causal, scale)
  torch.testing.assert_close(o.float(), o_ref, rtol=2e-2, atol=2e-2)
  torch.testing.assert_close(ctx[1], lse_ref, rtol=1e-3, atol=2e-3)


def test_flash_large_logits_rescale_path(kernel_lib):
  """Scores that grow along the keys force the running-max rescale of O."""
  from tunix_b200.ops import _lib, flash
  torch.manual_seed(1)
  B, L, N, H = 1, 512, 2, 128
  q = torch.randn(B, L, N, H, device="cuda").bfloat16()
  k = (torch.randn(B, L, N, H, device="cuda") * torch.linspace(0.5, 6.0, L, device="cuda")[None, :, None, None]).bfloat16()
  v = torch.randn(B, L, N, H, device="cuda").bfloat16()
  o, ctx = flash.forward(q, k, v, causal=True, scale=0.3)
  _lib.check_status()
  o_ref, lse_ref = ref_attention(q, k, v, True, 0.3)
  torch.testing.assert_close(o.float(), o_ref, rtol=3e-2, atol=3e-2)
  torch.testing.assert_close(ctx[1], lse_ref, rtol=1e-3, atol=5e-3)


@pytest.mark.parametrize("B,Lq,Lk,N,Kh,causal", [(2, 256, 256, 4, 2, True), (1, 128, 128, 1, 1, True),
                                                    (1, 200, 200, 4, 1, True), (1, 320, 320, 2, 2, False),
                                                    (1, 100, 333, 2, 1, True), (1, 1024, 1024, 8, 2, True)])
def test_flash_autograd_matches_reference(kernel_lib, B, Lq, Lk, N, Kh, causal):
  from tunix_b200.ops import _lib, flash
  torch.manual_seed(2)
  H = 128
  q = torch.randn(B, Lq, N, H, device="cuda").bfloat16().requires_grad_()
  k = torch.randn(B, Lk, Kh, H, device="cuda").bfloat16().requires_grad_()
  v = torch.randn(B, Lk, Kh, H, device="cuda").bfloat16().requires_grad_()
  o = flash.flash_attention(q, k, v, causal=causal, scale=0.09)
  g = torch.randn_like(o)
  o.backward(g)
  qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
  _lib.check_status()
  o_ref, _ = ref_attention(qf, kf, vf, causal, 0.09)
  o_ref.backward(g.float())
  for a, b in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
    torch.testing.assert_close(a.float(), b, rtol=5e-2, atol=5e-2)


def test_flash_backward_is_reproducible(kernel_lib):
  from tunix_b200.ops import flash
  torch.manual_seed(3)
  q, k, v = (torch.randn(1, 512, n, 128, device="cuda").bfloat16().requires_grad_() for n in (4, 2, 2))
  g = torch.randn(1, 512, 4, 128, device="cuda").bfloat16()
  grads = []
  for _ in range(2):
    for t in (q, k, v):
      t.grad = None
    flash.flash_attention(q, k, v, causal=True, scale=0.09).backward(g)
    grads.append([t.grad.clone() for t in (q, k, v)])
  for a, b in zip(*grads):
    assert torch.equal(a, b)


def _packed_ref(q, k, v, seg, causal, scale):
  """fp32 attention of packed rows: a token sees the tokens of its own segment (causally if asked)."""
  B, L, N, H = q.shape
  Kh = k.shape[2]
  qf = q.float().transpose(1, 2)
  kf = k.float().transpose(1, 2).repeat_interleave(N // Kh, 1)
  vf = v.float().transpose(1, 2).repeat_interleave(N // Kh, 1)
  s = qf @ kf.transpose(-1, -2) * scale
  vis = seg[:, :, None] == seg[:, None, :]
  if causal:
    vis = vis & torch.ones(L, L, dtype=torch.bool, device=q.device).tril()[None]
  s = s.masked_fill(~vis[:, None], float("-inf"))
  return (torch.softmax(s, -1) @ vf).transpose(1, 2)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("lengths", [[[100, 156]], [[64, 64, 128, 30, 226], [300, 212]], [[1, 700, 3, 320]]])
def test_flash_packed_segments_fwd_bwd(kernel_lib, lengths, causal):
  """Packed rows: segment boundaries inside and across tiles, forward and all three gradients."""
  from tunix_b200.ops import _lib, flash
  torch.manual_seed(3)
  B, L = len(lengths), sum(lengths[0])
  N, Kh, H = 4, 2, 128
  seg = torch.zeros(B, L, dtype=torch.int32, device="cuda")
  for b, ls in enumerate(lengths):
    assert sum(ls) == L
    pos = 0
    for i, n in enumerate(ls):
      seg[b, pos:pos + n] = i + 1
      pos += n
  q = torch.randn(B, L, N, H, device="cuda").bfloat16().requires_grad_()
  k = torch.randn(B, L, Kh, H, device="cuda").bfloat16().requires_grad_()
  v = torch.randn(B, L, Kh, H, device="cuda").bfloat16().requires_grad_()
  scale = 1.0 / math.sqrt(H)
  o = flash.flash_attention(q, k, v, causal=causal, scale=scale, segment_ids=seg)
  do = torch.randn_like(o)
  o.backward(do)
  _lib.check_status()
  got = (o.detach().float(), q.grad.float(), k.grad.float(), v.grad.float())
  qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
  o_ref = _packed_ref(qr, kr, vr, seg, causal, scale)
  o_ref.backward(do.float())
  want = (o_ref.detach(), qr.grad, kr.grad, vr.grad)
  for name, a, b in zip(("o", "dq", "dk", "dv"), got, want):
    err = (a - b).abs().max().item()
    assert err < 6e-2 * max(1.0, b.abs().max().item()), (name, err)


def test_packed_model_forward_matches_separate_sequences(kernel_lib):
  """A packed row through the decoder (fused layers, segment-aware flash) equals its sequences run alone."""
  from tunix_b200.models.transformer import ModelConfig, Transformer
  from tunix_b200.ops import _lib
  torch.manual_seed(5)
  cfg = ModelConfig(num_layers=2, vocab_size=512, embed_dim=256, hidden_dim=512, num_heads=2, head_dim=128,
                    num_kv_heads=1, dtype=torch.bfloat16, max_position=512)
  model = Transformer(cfg, device="cuda").init_weights(seed=0, scale=0.05)
  lens = [130, 62, 64]
  toks = [torch.randint(3, 512, (n,), device="cuda") for n in lens]
  packed = torch.cat(toks)[None]
  seg = torch.cat([torch.full((n,), i + 1, device="cuda", dtype=torch.int32) for i, n in enumerate(lens)])[None]
  pos = torch.cat([torch.arange(n, device="cuda") for n in lens])[None]
  for grad in (False, True):                     # the fused training node and the eager inference path
    with torch.set_grad_enabled(grad):
      logits, _ = model(packed, pos, None, None, segment_ids=seg)
      off = 0
      for t, n in zip(toks, lens):
        alone, _ = model(t[None], torch.arange(n, device="cuda")[None], None, None)
        torch.testing.assert_close(logits[0, off:off + n].float(), alone[0].float(), rtol=5e-2, atol=5e-2)
        off += n
  _lib.check_status()


def test_flash_packed_qkv_gradient_buffer_matches_separate_tensors(kernel_lib):
  """Attention straight from the fused [B, L, N + 2K, H] projection output: same output and the same gradient as the
  three-tensor form, with dq | dk | dv written into one buffer."""
  from tunix_b200.ops import flash
  torch.manual_seed(21)
  B, L, N, K, H = 2, 320, 8, 2, 128
  qkv = (torch.randn(B, L, N + 2 * K, H, device="cuda") * 0.5).to(torch.bfloat16)
  a = qkv.clone().requires_grad_()
  b = qkv.clone().requires_grad_()
  assert flash.packed_supported(a, N, K)
  oa = flash.flash_attention_packed(a, N, K, causal=True, scale=H ** -0.5)
  ob = flash.flash_attention(b[:, :, :N], b[:, :, N:N + K], b[:, :, N + K:], causal=True, scale=H ** -0.5)
  assert torch.equal(oa, ob)
  g = torch.randn_like(oa)
  oa.backward(g)
  ob.backward(g)
  assert torch.equal(a.grad, b.grad)
