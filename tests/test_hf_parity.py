"""Logit parity with Hugging Face transformers for every dense / MoE decoder family.

A tiny randomly initialised HF model is exported as a state dict, mapped through the safetensors
name rules into our decoder, and both run the same tokens in fp32 on the CPU. This checks RoPE
variants, norm conventions, GQA, qk-norm, soft-caps, sliding windows, tied heads and MoE routing
against an independent implementation.
"""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from tunix_b200.models import safetensors_loader
from tunix_b200.models.transformer import AttentionType, Transformer


def _ours(family, hf_cfg, **kw):
  from tunix_b200.models import registry
  mod = __import__(f"tunix_b200.models.{family}.model", fromlist=["ModelConfig"])
  base = dict(num_layers=hf_cfg.num_hidden_layers, vocab_size=hf_cfg.vocab_size, embed_dim=hf_cfg.hidden_size,
              hidden_dim=hf_cfg.intermediate_size, num_heads=hf_cfg.num_attention_heads,
              head_dim=getattr(hf_cfg, "head_dim", None) or hf_cfg.hidden_size // hf_cfg.num_attention_heads,
              num_kv_heads=hf_cfg.num_key_value_heads, norm_eps=hf_cfg.rms_norm_eps, dtype=torch.float32,
              max_position=64)
  base.update(kw)
  return mod.ModelConfig(**base)


def _compare(hf_model, cfg, atol=2e-4):
  hf_model = hf_model.eval().float()
  model = Transformer(cfg)
  state, unmatched = safetensors_loader.convert_state(
      hf_model.state_dict().items(), gemma_norms=str(cfg.family).startswith("gemma"))
  assert not [u for u in unmatched if "rotary" not in u and "inv_freq" not in u], unmatched
  params = dict(model.named_parameters())
  with torch.no_grad():
    for n, p in params.items():
      if n == "lm_head.w" and cfg.weight_tying:
        continue
      assert n in state, f"{n} missing from the converted checkpoint"
      assert tuple(state[n].shape) == tuple(p.shape), (n, state[n].shape, p.shape)
      p.copy_(state[n])
  torch.manual_seed(0)
  toks = torch.randint(0, cfg.vocab_size, (2, 24))
  with torch.no_grad():
    want = hf_model(toks).logits.float()
    got, _ = model(toks, torch.arange(24)[None].expand(2, 24), None, None)
  err = (got.float() - want).abs().max().item()
  assert err < atol * max(1.0, want.abs().max().item()), err


def _tiny(**kw):
  base = dict(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              vocab_size=128, max_position_embeddings=64, rms_norm_eps=1e-6, attention_dropout=0.0)
  base.update(kw)
  return base


def test_llama_parity():
  from transformers import LlamaConfig, LlamaForCausalLM
  hf = LlamaConfig(**_tiny(rope_theta=500000.0, tie_word_embeddings=False))
  torch.manual_seed(1)
  _compare(LlamaForCausalLM(hf), _ours("llama3", hf, rope_theta=500000.0, weight_tying=False))


def test_qwen2_parity_with_biases():
  from transformers import Qwen2Config, Qwen2ForCausalLM
  hf = Qwen2Config(**_tiny(rope_theta=1000000.0, tie_word_embeddings=True))
  torch.manual_seed(2)
  m = Qwen2ForCausalLM(hf)
  with torch.no_grad():
    for n, p in m.named_parameters():
      if n.endswith("bias"):
        p.normal_(0, 0.1)
  _compare(m, _ours("qwen2", hf, rope_theta=1000000.0, weight_tying=True))


def test_qwen3_parity_with_qk_norm():
  from transformers import Qwen3Config, Qwen3ForCausalLM
  hf = Qwen3Config(**_tiny(head_dim=32, rope_theta=1000000.0, tie_word_embeddings=False))
  torch.manual_seed(3)
  m = Qwen3ForCausalLM(hf)
  with torch.no_grad():
    for n, p in m.named_parameters():
      if "q_norm" in n or "k_norm" in n:
        p.uniform_(0.5, 1.5)
  _compare(m, _ours("qwen3", hf, rope_theta=1000000.0, weight_tying=False))


def test_qwen3_moe_parity():
  from transformers import Qwen3MoeConfig, Qwen3MoeForCausalLM
  hf = Qwen3MoeConfig(**_tiny(head_dim=32, rope_theta=1000000.0, tie_word_embeddings=False, num_experts=4,
                              num_experts_per_tok=2, moe_intermediate_size=48, norm_topk_prob=True,
                              decoder_sparse_step=1, mlp_only_layers=[]))
  torch.manual_seed(4)
  _compare(Qwen3MoeForCausalLM(hf), _ours("qwen3", hf, rope_theta=1000000.0, weight_tying=False, num_experts=4,
                                         num_experts_per_tok=2, moe_hidden_dim=48, hidden_dim=48, norm_topk_prob=True),
           atol=5e-4)


def test_gemma2_parity_softcaps_and_sliding_window():
  from transformers import Gemma2Config, Gemma2ForCausalLM
  hf = Gemma2Config(**_tiny(head_dim=16, rope_theta=10000.0, query_pre_attn_scalar=16, sliding_window=8,
                            attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
                            hidden_activation="gelu_pytorch_tanh", attn_implementation="eager"))
  torch.manual_seed(5)
  m = Gemma2ForCausalLM(hf)
  with torch.no_grad():
    for n, p in m.named_parameters():
      if "norm" in n:
        p.normal_(0, 0.2)
  _compare(m, _ours("gemma", hf, rope_theta=10000.0, sliding_window_size=8, attn_logits_soft_cap=50.0,
                    final_logit_softcap=30.0, use_post_attn_norm=True, use_post_ffw_norm=True,
                    attention_types=(AttentionType.LOCAL_SLIDING, AttentionType.GLOBAL)), atol=5e-4)


def test_gemma3_text_parity_local_global_rope():
  from transformers import Gemma3TextConfig, Gemma3ForCausalLM
  hf = Gemma3TextConfig(**_tiny(head_dim=16, num_hidden_layers=6, query_pre_attn_scalar=16, sliding_window=8,
                                rope_theta=1000000.0, rope_local_base_freq=10000.0,
                                hidden_activation="gelu_pytorch_tanh", attn_implementation="eager"))
  torch.manual_seed(6)
  m = Gemma3ForCausalLM(hf)
  with torch.no_grad():
    for n, p in m.named_parameters():
      if "norm" in n:
        p.normal_(0, 0.2)
  _compare(m, _ours("gemma3", hf, sliding_window_size=8), atol=5e-4)


def test_gemma3_multimodal_parity_vision_tower_projector_and_merge():
  """SigLIP tower + average pooling + soft-embedding norm + projector + merge into the text embeddings, against
  Hugging Face `Gemma3ForConditionalGeneration` with the same random weights (plain causal mask on both sides)."""
  from transformers import Gemma3Config, Gemma3ForConditionalGeneration, Gemma3TextConfig, SiglipVisionConfig
  from tunix_b200.models.gemma3 import vision as vis
  tc = Gemma3TextConfig(**_tiny(head_dim=16, query_pre_attn_scalar=16, sliding_window=32, rope_theta=1000000.0,
                                rope_local_base_freq=10000.0, hidden_activation="gelu_pytorch_tanh",
                                attn_implementation="eager"))
  vc = SiglipVisionConfig(hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=2,
                          image_size=28, patch_size=7, num_channels=3, attn_implementation="eager")
  cfg = Gemma3Config(text_config=tc, vision_config=vc, mm_tokens_per_image=4, image_token_index=5, boi_token_index=6,
                     eoi_token_index=7, attn_implementation="eager")
  torch.manual_seed(9)
  hf = Gemma3ForConditionalGeneration(cfg).eval().float()
  with torch.no_grad():
    for n, p in hf.named_parameters():
      if "norm" in n and p.dim() == 1:
        p.normal_(0, 0.2) if "vision" not in n else p.add_(torch.randn_like(p) * 0.1)
  ours_text = Transformer(_ours("gemma3", tc, sliding_window_size=32))
  vcfg = vis.SigLIPConfig(num_mm_tokens_per_image_prepool=16, num_mm_tokens_per_image=4, image_height=28, image_width=28,
                          soft_token_placeholder=5, patch_size=(7, 7), width=32, depth=2, mlp_dim=48, num_heads=2)
  model = vis.Gemma3Multimodal(ours_text, vcfg, dtype=torch.float32).eval()
  unused = vis.load_hf_multimodal_state(model, hf.state_dict().items())
  assert all("head." in u or "rotary" in u or "inv_freq" in u for u in unused), unused
  toks = torch.randint(8, 128, (2, 20))
  toks[:, 3:7] = 5                                       # one image of 4 soft tokens per row
  pixels = torch.randn(2, 3, 28, 28)
  L = toks.shape[1]
  causal = torch.ones(L, L, dtype=torch.bool).tril()[None].expand(2, L, L)
  with torch.no_grad():
    want = hf(input_ids=toks, pixel_values=pixels).logits.float()
    got, _ = model(toks, torch.arange(L)[None].expand(2, L), None, causal,
                   images=pixels.permute(0, 2, 3, 1)[:, None])      # [B, N=1, H, W, C]
  err = (got.float() - want).abs().max().item()
  assert err < 5e-4 * max(1.0, want.abs().max().item()), err
