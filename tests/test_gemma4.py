"""Gemma 4 text decoder: layer pattern, KV sharing, per-layer inputs, partial RoPE, MoE branch, cache."""
import torch

from tunix_b200.models.gemma4 import AttentionType, Gemma4, ModelConfig, kv_sharing_pattern
from tunix_b200.models.gemma4 import model as g4


def tiny(**kw):
  base = dict(num_layers=7, num_embed=64, embed_dim=32, hidden_dim=48, num_heads=4, head_dim=8, num_kv_heads=2,
              sliding_window_size=4, per_layer_input_dim=6, frac_shared_layers=4.0 / 7, global_key_size=16,
              num_global_kv_heads=1, k_eq_v_global=True, override_kv_shared_ffw_hidden=64,
              attention_pattern=(AttentionType.LOCAL_SLIDING, AttentionType.LOCAL_SLIDING, AttentionType.GLOBAL))
  base.update(kw)
  return ModelConfig(**base)


def test_presets_and_sharing_pattern():
  c = ModelConfig.gemma4_e2b()
  types = c.attention_types()
  assert len(types) == 35 and types[4] == AttentionType.GLOBAL and types[3] == AttentionType.LOCAL_SLIDING
  pat = kv_sharing_pattern(35, 20.0 / 35, types)
  assert pat[:15] == list(range(15))
  assert all(pat[i] == (14 if types[i] == AttentionType.GLOBAL else 13) for i in range(15, 35))
  assert types[14] == AttentionType.GLOBAL and types[13] == AttentionType.LOCAL_SLIDING
  assert ModelConfig.gemma4_26b_a4b_it().num_experts == 128 and ModelConfig.gemma4_31b().num_global_kv_heads == 4


def test_structure_of_shared_and_global_layers():
  m = Gemma4(tiny())
  # pattern L L G | L L G L: three unshared layers, the four after them reuse layer 2 (global) or 1 (local)
  assert m.kv_sharing == [0, 1, 2, 1, 1, 2, 1]
  for i in range(3, 7):
    assert m.layers[i].attn.k_proj is None
    assert m.layers[i].mlp.down_proj.shape[1] == 64          # wider MLP on shared layers
  glob = m.layers[2].attn
  assert glob.head_dim == 16 and glob.num_kv_heads == 1 and glob.v_proj is None       # k == v on global layers
  assert m.layers[0].attn.head_dim == 8 and m.layers[0].attn.v_proj is not None


def test_partial_rope_rotates_only_the_leading_pairs():
  x = torch.randn(1, 5, 2, 16)
  pos = torch.arange(5)[None]
  y = g4.partial_rope(x, pos, 10000.0, 1.0, 0.25)          # 2 of 8 pairs rotate
  assert torch.allclose(y[..., 2:8], x[..., 2:8]) and torch.allclose(y[..., 10:], x[..., 10:])
  assert not torch.allclose(y[0, 1:, :, :2], x[0, 1:, :, :2])
  assert torch.allclose(y[0, 0], x[0, 0])                   # position 0 is the identity
  full = g4.partial_rope(x, pos, 10000.0, 1.0, 1.0)
  assert torch.allclose(full.norm(dim=-1), x.norm(dim=-1), atol=1e-5)


def test_cached_decode_matches_full_forward_and_gradients_flow():
  torch.manual_seed(0)
  for moe in (False, True):
    kw = dict(enable_moe=True, num_experts=4, num_experts_per_tok=2, expert_dim=24) if moe else {}
    m = Gemma4(tiny(**kw)).init_weights(seed=1, scale=0.2)
    toks = torch.randint(0, 64, (2, 9))
    full, _ = m(toks)
    assert full.shape == (2, 9, 64) and float(full.abs().max()) <= 30.0
    # prefill 5 tokens into a cache, then 4 single-token steps
    cache = m.init_cache(2, 16)
    assert set(cache) == {"layer_0", "layer_1", "layer_2"}
    pos = torch.arange(9)[None].expand(2, 9)
    out, cache = m(toks[:, :5], pos[:, :5], cache, None)
    steps = [out]
    for t in range(5, 9):
      o, cache = m(toks[:, t:t + 1], pos[:, t:t + 1], cache, None)
      steps.append(o)
    assert torch.allclose(torch.cat(steps, 1), full, atol=2e-4), float((torch.cat(steps, 1) - full).abs().max())
    full.square().mean().backward()
    missing = [n for n, p in m.named_parameters() if p.grad is None]
    assert not missing, missing


def test_sliding_window_limits_what_a_local_layer_sees():
  torch.manual_seed(1)
  cfg = tiny(num_layers=1, frac_shared_layers=0.0, per_layer_input_dim=0,
             attention_pattern=(AttentionType.LOCAL_SLIDING,), sliding_window_size=3)
  m = Gemma4(cfg).init_weights(seed=2, scale=0.3)
  a = torch.randint(0, 64, (1, 8))
  b = a.clone()
  b[0, 0] = (a[0, 0] + 1) % 64                 # differs only at position 0
  ya, _ = m(a)
  yb, _ = m(b)
  assert not torch.allclose(ya[0, 2], yb[0, 2])     # position 2 still sees position 0 (window 3)
  assert torch.allclose(ya[0, 3:], yb[0, 3:], atol=1e-6)   # positions >= 3 do not


def test_automodel_builds_a_random_gemma4():
  from tunix_b200.models import automodel
  cfg = tiny()
  m, path = automodel.AutoModel.from_pretrained("google/gemma-4-e2b-it", model_source=automodel.ModelSource.DUMMY,
                                                model_config=cfg, dtype=torch.float32, device="cpu")
  assert isinstance(m, Gemma4) and path is None
  logits, _ = m(torch.randint(0, 64, (1, 5)))
  assert logits.shape == (1, 5, 64) and bool(torch.isfinite(logits).all())


# ------------------------------------------------------------------------------------------ vision tower
def _grid_positions(cols, rows, pad_to):
  xy = [(c, r) for r in range(rows) for c in range(cols)]
  xy += [(-1, -1)] * (pad_to - len(xy))
  return torch.tensor(xy)


def test_vision_pieces_against_plain_restatements():
  from tunix_b200.models.gemma4 import vision as v
  torch.manual_seed(0)
  # factorised position embedding = one-hot contraction over both coordinates
  table = torch.randn(6, 2, 5)
  pos = torch.stack([_grid_positions(3, 2, 8), _grid_positions(2, 3, 8)])
  got = v.factorized_posemb(table, pos)
  onehot = torch.nn.functional.one_hot(pos.clamp(min=0), 6).float() * (pos >= 0)[..., None]
  want = torch.einsum("blis,sid->bld", onehot, table)
  assert torch.allclose(got, want, atol=1e-6) and got[0, 7].abs().sum() == 0
  assert torch.isnan(v.factorized_posemb(table, torch.tensor([[[9, 0]]]))).all()
  # pooling by coordinates: a 4 x 2 grid (+ padding) pooled 2 x 2 into 2 cells (of 3 slots)
  x = torch.randn(1, 12, 4)
  p = _grid_positions(4, 2, 12)[None]
  pooled, mask = v.avg_pool_by_positions(x, p, 3)
  cell0 = x[0, [0, 1, 4, 5]].mean(0)
  cell1 = x[0, [2, 3, 6, 7]].mean(0)
  assert torch.allclose(pooled[0, 0], cell0, atol=1e-6) and torch.allclose(pooled[0, 1], cell1, atol=1e-6)
  assert mask.tolist() == [[True, True, False]] and pooled[0, 2].abs().sum() == 0
  # 2-D rotary: norm-preserving, identity at the origin, first half depends on x only, second half on y only
  h = torch.randn(1, 3, 2, 8)
  xy = torch.tensor([[[0, 0], [3, 0], [0, 5]]])
  r = v.rope_2d(h, xy)
  assert torch.allclose(r.norm(dim=-1), h.norm(dim=-1), atol=1e-5) and torch.allclose(r[0, 0], h[0, 0])
  assert torch.allclose(r[0, 1, :, 4:], h[0, 1, :, 4:]) and not torch.allclose(r[0, 1, :, :4], h[0, 1, :, :4])
  assert torch.allclose(r[0, 2, :, :4], h[0, 2, :, :4]) and not torch.allclose(r[0, 2, :, 4:], h[0, 2, :, 4:])
  # relative property: <rope(q, p), rope(k, p')> depends on p - p' only
  q, k = torch.randn(1, 1, 1, 8), torch.randn(1, 1, 1, 8)
  dot = lambda a, b: (v.rope_2d(q, torch.tensor([[a]])) * v.rope_2d(k, torch.tensor([[b]]))).sum()
  assert torch.allclose(dot([5, 7], [2, 3]), dot([4, 9], [1, 5]), atol=1e-4)


def test_vision_encoder_ignores_padding_and_feeds_the_decoder():
  from tunix_b200.models.gemma4 import vision as v
  torch.manual_seed(1)
  vc = v.VisionEncoderConfig(d_model=16, num_layers=2, num_heads=2, ffw_hidden=32, patch_size=2, output_length=4,
                             pos_emb_shape_yx=(16, 2), pooling_kernel_size=2, standardize_embeddings=True)
  assert vc.max_patches == 16 and vc.image_height == 8
  enc = v.VisionEncoder(vc).init_weights(seed=2, scale=0.2)
  patches = torch.rand(2, 16, 12)
  pos = torch.stack([_grid_positions(4, 4, 16), _grid_positions(4, 2, 16)])           # the second image is half size
  (emb, mask), = enc(patches, pos)
  assert emb.shape == (2, 4, 16) and mask.tolist() == [[True] * 4, [True, True, False, False]]
  # padding content does not leak into valid outputs
  noisy = patches.clone()
  noisy[1, 8:] = torch.rand(8, 12) * 50
  (emb2, _), = enc(noisy, pos)
  assert torch.allclose(emb2[1, :2], emb[1, :2], atol=1e-5) and torch.allclose(emb2[0], emb[0], atol=1e-5)
  # clipped linears: finite bounds clamp, infinite ones are the plain linear
  lin = v.ClippedLinear(3, 4, True, torch.float32)
  with torch.no_grad():
    lin.w.copy_(torch.ones(3, 4))
  xx = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
  assert lin(xx).tolist() == [[10.0] * 3]
  lin.clip_input_max.fill_(2.0); lin.clip_output_max.fill_(6.5)
  assert lin(xx).tolist() == [[6.5] * 3]
  seg = v.ClippedLinear((1, 2), 4, True, torch.float32)               # two segments with their own clamps
  with torch.no_grad():
    seg.w.copy_(torch.ones(3, 4))
  seg.clip_input_max[1] = 1.0; seg.clip_output_min[0] = 20.0
  assert seg(xx).tolist() == [[20.0, 4.0, 4.0]]

  # decoder side: placeholders are replaced in order, each row by its own images; text positions untouched
  cfg = tiny(vision_encoder=vc, use_bidirectional_attention="vision")
  model = Gemma4(cfg).init_weights(seed=3, scale=0.1)
  with torch.no_grad():
    model.vision_encoder.load_state_dict(enc.state_dict())
  I = g4.IMAGE_SOFT_TOKEN_PLACEHOLDER
  tokens = torch.tensor([[5, I, I, I, I, 6, 7, 8], [9, I, I, 10, 11, 12, 13, 14]])
  images = v.PreprocessedVisionInput(patches=patches, positions_xy=pos, soft_token_counts=[[4], [2]])
  x_text = model.embedder.encode(tokens)
  x = model._merge_modalities(x_text, tokens, images, None)
  proj = model.embedder.encode_vision(emb)
  assert torch.allclose(x[0, 1:5], proj[0], atol=1e-5) and torch.allclose(x[1, 1:3], proj[1, :2], atol=1e-5)
  assert torch.equal(x[0, 5:], x_text[0, 5:]) and torch.equal(x[1, 3:], x_text[1, 3:]) and torch.equal(x[:, 0], x_text[:, 0])
  causal = torch.ones(8, 8, dtype=torch.bool).tril()[None].expand(2, 8, 8)
  opened = g4.add_bidirectional_blocks(causal, tokens == I)
  assert opened[0, 1, 4] and opened[0, 2, 3] and not opened[0, 0, 1] and not opened[0, 5, 6] and not opened[1, 1, 3]
  logits, _ = model(tokens, None, None, causal, images=images)
  logits_text, _ = model(tokens, None, None, causal)
  assert logits.shape == (2, 8, 64) and torch.isfinite(logits).all()
  assert not torch.allclose(logits[0, 5], logits_text[0, 5])              # later text positions see the image
  assert torch.allclose(logits[0, 0], logits_text[0, 0], atol=1e-5)       # earlier ones do not


# ------------------------------------------------------------------------------------------ audio tower
def _blocked_local_attention(att, x, mask, block=4):
  """The block formulation: queries in blocks of `block`, keys gathered with left context per block, relative
  logits aligned by the pad-and-reshape shift, band + validity mask per block. Oracle for the band kernel."""
  import math
  from tunix_b200.models.gemma4 import audio as a
  B, T, _ = x.shape
  N, H, L = att.N, att.H, att.L
  q, k, v = (proj(x).float().view(B, T, N, H) for proj in att.qkv)
  q = q * (a._R_SOFTPLUS_0 / math.sqrt(H)) * torch.nn.functional.softplus(att.per_dim_scale.float())
  k = k * (a._R_SOFTPLUS_0 * math.log1p(math.e))
  U = (T + block - 1) // block
  C = block + L

  def ctx(t, fill):
    tp = torch.nn.functional.pad(t.float(), [0, 0] * (t.dim() - 2) + [L, block - 1], value=fill)
    idx = (torch.arange(U) * block)[:, None] + torch.arange(C)[None, :]
    return tp[:, idx]

  qb = torch.nn.functional.pad(q, [0, 0, 0, 0, 0, U * block - T]).view(B, U, block, N, H)
  kb, vb = ctx(k, 0.0), ctx(v, 0.0)
  ac = torch.einsum("buwnh,bucnh->bnuwc", qb, kb)
  E = torch.nn.functional.linear(a.sinusoid(torch.arange(L, -1, -1), N * H), att.pos_proj.float()).view(L + 1, N, H)
  bd = torch.einsum("buwnh,fnh->bnuwf", qb, E)
  bd = torch.nn.functional.pad(bd, (0, (C + 1) - (L + 1))).reshape(B, N, U, block * (C + 1))[..., :block * C]
  logits = a._SOFTCAP * torch.tanh((ac + bd.view(B, N, U, block, C)) / a._SOFTCAP)
  w_, c_ = torch.arange(block)[:, None], torch.arange(C)[None, :]
  band = (c_ >= w_) & (c_ - w_ <= L)
  valid = ctx(mask, 0.0).bool()[:, None, :, None, :] & band[None, None, None]
  probs = torch.softmax(torch.where(valid, logits, torch.full_like(logits, -1e9)), dim=-1)
  out = torch.einsum("bnuwc,bucnh->buwnh", probs, vb)
  return out.reshape(B, U * block, N, H)[:, :T]


def test_audio_front_end_and_band_attention():
  import numpy as np
  from tunix_b200.models.gemma4 import audio as a
  torch.manual_seed(0)
  mel = a.MelFilterbank()
  wave = torch.randn(2, 16000) * 0.1
  got = mel(wave)
  assert got.shape == (2, mel.num_frames(16000), 128) and mel.num_frames(16000) == 98 and mel.num_frames(320) == 0
  # first frame, spelled out: 320 samples x window -> 512-point spectrum magnitude -> triangles -> log
  frame = wave[0, :320].numpy() * mel.window.numpy()
  spec = np.abs(np.fft.rfft(frame, n=512))
  assert np.allclose(got[0, 0].numpy(), np.log(spec @ mel.mel_basis.numpy() + 1e-3), atol=1e-4)
  assert mel.window.min() > 0 and (mel.mel_basis >= 0).all() and float(mel.mel_basis.max()) <= 1.0
  assert a.to_float32(torch.tensor([16384], dtype=torch.int16)).item() == 0.5

  cfg = a.ConformerConfig(num_layers=2, model_dims=32, lm_model_dims=24, atten_num_heads=4, atten_left_context=6,
                          conv_kernel_size=3)
  att = a.BandAttention(cfg, torch.float32)
  with torch.no_grad():
    for p in att.parameters():
      p.copy_(torch.randn(p.shape) * 0.3)
  x = torch.randn(2, 11, 32)
  mask = torch.ones(2, 11, dtype=torch.bool)
  mask[1, 7:] = False
  band = att(x, mask)
  for block in (4, 12):
    ref = _blocked_local_attention(att, x, mask, block=block)
    assert torch.allclose(band[0], ref[0], atol=1e-5) and torch.allclose(band[1, :7], ref[1, :7], atol=1e-5)
  # a frame never sees beyond its left context nor the future
  x2 = x.clone()
  x2[0, 0] += 5.0
  x2[0, 10] += 5.0
  moved = (att(x2, mask)[0] - band[0]).abs().amax(dim=(-1, -2)) > 1e-6
  assert moved.tolist() == [True] * 6 + [False] * 4 + [True]


def test_audio_tokenizer_lengths_padding_and_decoder_merge():
  from tunix_b200.models.gemma4 import audio as a, vision as v
  torch.manual_seed(1)
  cfg = a.ConformerConfig(num_layers=2, model_dims=32, lm_model_dims=24, atten_num_heads=4, atten_left_context=5,
                          conv_kernel_size=3)
  tok = a.AudioTokenizer(cfg).init_weights(seed=4, scale=0.2)
  samples = 4000
  waves = torch.randn(2, samples) * 0.1
  lengths = torch.tensor([samples, 2400])
  emb, pad = tok(waves, lengths)
  assert emb.shape == (2, tok.get_num_soft_tokens(samples), 24) and tok.get_num_soft_tokens(100) == 0
  assert not pad[0].any() and pad[1].sum() > 0 and emb[1][pad[1]].abs().sum() == 0
  n_valid = int((~pad[1]).sum())
  assert abs(n_valid - tok.get_num_soft_tokens(2400)) <= 1
  # what lies beyond a clip's length does not change its earlier tokens (streaming model: past-only context)
  noisy = waves.clone()
  noisy[1, 2400:] = torch.randn(samples - 2400) * 3
  emb2, pad2 = tok(noisy, lengths)
  assert torch.equal(pad, pad2) and torch.allclose(emb2[1, :n_valid - 2], emb[1, :n_valid - 2], atol=1e-4)

  model_cfg = tiny(audio_encoder=cfg)
  model = Gemma4(model_cfg).init_weights(seed=5, scale=0.1)
  with torch.no_grad():
    model.audio_encoder.load_state_dict(tok.state_dict())
  A = g4.AUDIO_SOFT_TOKEN_PLACEHOLDER
  T = emb.shape[1]
  tokens = torch.tensor([[5] + [A] * T + [6, 7], [9] + [A] * n_valid + [3] * (T - n_valid) + [10, 11]])
  audios = a.PreprocessedAudioInput(audios=waves[:, None], sequence_lengths=lengths[:, None])
  x_text = model.embedder.encode(tokens)
  x = model._merge_modalities(x_text, tokens, None, audios)
  want = model.embedder.encode_audio(emb)
  assert torch.allclose(x[0, 1:1 + T], want[0], atol=1e-5) and torch.allclose(x[1, 1:1 + n_valid], want[1, :n_valid], atol=1e-5)
  assert torch.equal(x[1, 1 + n_valid:], x_text[1, 1 + n_valid:])
  logits, _ = model(tokens, None, None, None, audios=audios)
  assert torch.isfinite(logits).all() and logits.shape[:2] == tokens.shape


def test_checkpoint_names_round_trip_for_text_vision_audio(tmp_path):
  from tunix_b200.models.gemma4 import audio as a, params_safetensors as ps, vision as v
  torch.manual_seed(3)
  vc = v.VisionEncoderConfig(d_model=16, num_layers=2, num_heads=2, ffw_hidden=32, patch_size=2, output_length=4,
                             pos_emb_shape_yx=(16, 2), pooling_kernel_size=2, standardize_embeddings=True,
                             use_clipped_linears=True)
  ac = a.ConformerConfig(num_layers=2, model_dims=32, lm_model_dims=24, atten_num_heads=4, atten_left_context=5,
                         conv_kernel_size=3)
  cfg = tiny(vision_encoder=vc, audio_encoder=ac, enable_moe=True, num_experts=4, num_experts_per_tok=2, expert_dim=16)
  src = Gemma4(cfg)
  with torch.no_grad():
    for t in src.state_dict().values():
      t.copy_(torch.randn(t.shape) if t.is_floating_point() else t)
  # in a checkpoint v shares k's clamps and up shares gate's: make the source consistent with that
  for blk in src.vision_encoder.layers:
    for name in ("clip_input_min", "clip_input_max", "clip_output_min", "clip_output_max"):
      getattr(blk.attn.qkv_proj, name)[2] = getattr(blk.attn.qkv_proj, name)[1]
      getattr(blk.mlp.gate_up_proj, name)[1] = getattr(blk.mlp.gate_up_proj, name)[0]
  hf = ps.to_hf(cfg, src.state_dict())
  assert "model.language_model.layers.0.mlp.gate_proj.weight" in hf and "model.language_model.layers.3.self_attn.q_proj.weight" in hf
  assert "model.language_model.layers.3.self_attn.k_proj.weight" not in hf          # layer 3 shares K/V
  assert hf["model.vision_tower.patch_embedder.position_embedding_table"].shape == (2, 16, 16)
  assert "model.vision_tower.encoder.layers.1.self_attn.k_proj.input_max" in hf
  assert "model.vision_tower.encoder.layers.1.self_attn.v_proj.input_max" not in hf
  assert hf["model.audio_tower.layers.1.self_attn.post.linear.weight"].shape == (32, 32)
  assert hf["model.language_model.layers.0.experts.gate_up_proj"].shape == (4, 32, 32)
  path = ps.save_checkpoint(src, str(tmp_path))
  assert path.endswith("model.safetensors")
  dst = ps.load_checkpoint(Gemma4(cfg), str(tmp_path))
  for (n, p), (_, q) in zip(src.state_dict().items(), dst.state_dict().items()):
    assert torch.equal(p, q), n
  # keys without the prefixes load as well; a missing tensor is named
  bare = {k.replace("model.language_model.", "").replace("model.", ""): t for k, t in hf.items()}
  again = ps.from_hf(cfg, bare, src.state_dict().keys())
  assert torch.equal(again["layers.2.mlp.gate_up_proj"], src.state_dict()["layers.2.mlp.gate_up_proj"])
  del bare["norm.weight"]
  try:
    ps.from_hf(cfg, bare, src.state_dict().keys())
    raise AssertionError("expected KeyError")
  except KeyError as e:
    assert "final_norm" in str(e)


def test_window_sized_ring_cache_matches_the_full_cache():
  """Local layers that keep only `sliding_window_size` keys give the same logits as a full-length cache: a prompt
  longer than the window, then decode steps that wrap the ring several times; shared layers read the ring too."""
  torch.manual_seed(5)
  full_cfg, ring_cfg = tiny(), tiny(use_sliding_window_kv_cache=True)
  full = Gemma4(full_cfg).init_weights(seed=7, scale=0.2)
  ring = Gemma4(ring_cfg).init_weights(seed=7, scale=0.2)
  B, P, steps, size = 2, 7, 9, 24
  tokens = torch.randint(1, 60, (B, P + steps))
  cf, cr = full.init_cache(B, size), ring.init_cache(B, size)
  assert cr["layer_0"]["k"].shape[1] == 4 and cr["layer_2"]["k"].shape[1] == size and cf["layer_0"]["k"].shape[1] == size
  pos = torch.arange(P)[None].expand(B, P)
  causal = torch.ones(P, size, dtype=torch.bool).tril()[None].expand(B, P, size)
  lf, cf = full(tokens[:, :P], pos, cf, causal)
  lr, cr = ring(tokens[:, :P], pos, cr, causal)
  assert torch.allclose(lf, lr, atol=1e-5)
  for t in range(P, P + steps):
    step_mask = (torch.arange(size) <= t)[None, None, :].expand(B, 1, size)
    p1 = torch.full((B, 1), t)
    lf, cf = full(tokens[:, t:t + 1], p1, cf, step_mask)
    lr, cr = ring(tokens[:, t:t + 1], p1, cr, step_mask)
    assert torch.allclose(lf, lr, atol=1e-5), t
  assert int(cr["layer_0"]["end_index"][0]) == P + steps
