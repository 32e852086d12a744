"""Naming, registry, safetensors round trips, LoRA-merged export, AutoModel."""
import dataclasses
import json
import os

import pytest
import torch

from tunix_b200.models import automodel, dummy_model_creator, lora, naming, registry, safetensors_io
from tunix_b200.models import safetensors_loader, safetensors_saver
from tunix_b200.models.transformer import Transformer


def tiny(family_mod, preset, **kw):
  cfg = getattr(family_mod.ModelConfig, preset)()
  base = dict(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=4, head_dim=8, num_kv_heads=2)
  if cfg.num_experts:
    base.update(num_experts=4, num_experts_per_tok=2, moe_hidden_dim=16, hidden_dim=16)
  base.update(kw)
  return dataclasses.replace(cfg, **base)


def test_naming_rules():
  n = naming.ModelNaming(model_id="meta-llama/Llama-3.1-8B")
  assert (n.model_name, n.model_family, n.model_version, n.model_config_category, n.model_config_id) == \
      ("llama-3.1-8b", "llama3p1", "8b", "llama3", "llama3p1_8b")
  assert naming.ModelNaming(model_id="google/gemma-2-2b-it").model_config_id == "gemma2_2b_it"
  assert naming.ModelNaming(model_name="qwen2.5-0.5b").model_config_id == "qwen2p5_0p5b"
  assert naming.ModelNaming(model_id="qwen3_30b_a3b").model_family == "qwen3"
  with pytest.raises(ValueError):
    naming.ModelNaming(model_id="acme/unknown-7b")
  with pytest.raises(ValueError):
    naming.ModelNaming(model_id="Qwen/Qwen3-8B", model_family="llama3")
  with pytest.raises(ValueError):
    naming.ModelNaming()


def test_registry_covers_presets():
  ids = registry.config_ids()
  for want in ("llama3p1_8b", "qwen3_8b", "qwen3_30b_a3b", "gemma2_2b_it", "qwen2p5_0p5b"):
    assert want in ids
  assert registry.lookup("Qwen/Qwen3-8B").model_config_id == "qwen3_8b"
  cfg = automodel.call_model_config("llama-3.1-8b")
  assert cfg.num_layers == 32 and cfg.embed_dim == 4096 and cfg.vocab_size == 128256


def test_safetensors_io_round_trip(tmp_path):
  t = {"a": torch.randn(3, 4), "b": torch.arange(6, dtype=torch.int64).view(2, 3), "c": torch.randn(5).bfloat16(),
       "e": torch.empty(0, 4)}
  p = str(tmp_path / "x.safetensors")
  safetensors_io.save_file(t, p, metadata={"format": "pt"})
  f = safetensors_io.SafeTensorsFile(p)
  assert sorted(f.keys()) == ["a", "b", "c", "e"] and f.metadata == {"format": "pt"}
  for k in t:
    assert torch.equal(f.get(k), t[k])
  try:
    import safetensors.torch as st
    ref = st.load_file(p)
    for k in t:
      assert torch.equal(ref[k], t[k])
  except ImportError:
    pass


@pytest.mark.parametrize("family,preset", [("llama3", "llama3p1_8b"), ("qwen3", "qwen3_8b"), ("qwen2", "qwen2p5_0p5b"),
                                           ("gemma", "gemma2_2b"), ("qwen3", "qwen3_30b_a3b")])
def test_hf_export_import_round_trip(tmp_path, family, preset):
  import importlib
  mod = importlib.import_module(f"tunix_b200.models.{family}.model")
  cfg = tiny(mod, preset)
  m = Transformer(cfg).init_weights(seed=3, scale=0.1)
  out = safetensors_saver.save_lora_merged_model_as_safetensors(None, str(tmp_path), m)
  keys = safetensors_io.SafeTensorsFile(out).keys()
  assert "model.layers.0.self_attn.q_proj.weight" in keys and "model.embed_tokens.weight" in keys
  if cfg.num_experts:
    assert "model.layers.1.mlp.experts.3.down_proj.weight" in keys and "model.layers.0.mlp.gate.weight" in keys
  m2 = Transformer(cfg).init_weights(seed=9, scale=0.1)
  ignored = safetensors_loader.load_into_model(m2, str(tmp_path))
  assert ignored == []
  for (n1, p1), (n2, p2) in zip(m.named_parameters(), m2.named_parameters()):
    assert n1 == n2 and torch.equal(p1, p2), n1
  tok = torch.randint(0, 64, (2, 6))
  pos = torch.arange(6)[None].expand(2, -1)
  mask = torch.tril(torch.ones(6, 6, dtype=torch.bool))[None].expand(2, -1, -1)
  torch.testing.assert_close(m(tok, pos, None, mask)[0], m2(tok, pos, None, mask)[0])


def test_lora_merged_export_matches_adapter_forward(tmp_path):
  from tunix_b200.models.llama3 import model as llama
  cfg = tiny(llama, "llama3p2_1b")
  m = Transformer(cfg).init_weights(seed=1, scale=0.1)
  lora.apply_lora_to_model(m, rank=4, alpha=8.0, module_path=".*q_proj|.*v_proj|.*down_proj")
  with torch.no_grad():
    for n, p in m.named_parameters():
      if getattr(p, "is_lora", False):
        p.normal_(0, 0.1)
  safetensors_saver.save_lora_merged_model_as_safetensors(None, str(tmp_path), m)
  assert lora.is_lora_enabled(m)      # export leaves the adapters in place
  plain = Transformer(cfg)
  safetensors_loader.load_into_model(plain, str(tmp_path))
  tok = torch.randint(0, 64, (2, 6))
  pos = torch.arange(6)[None].expand(2, -1)
  mask = torch.tril(torch.ones(6, 6, dtype=torch.bool))[None].expand(2, -1, -1)
  torch.testing.assert_close(m(tok, pos, None, mask)[0], plain(tok, pos, None, mask)[0], rtol=1e-4, atol=1e-4)


def test_automodel_dummy_and_local_path(tmp_path):
  from tunix_b200.models.qwen3 import model as qwen3
  cfg = tiny(qwen3, "qwen3_0p6b")
  m, path = automodel.AutoModel.from_pretrained("Qwen/Qwen3-0.6B", model_source=automodel.ModelSource.DUMMY,
                                                model_config=cfg, dtype=torch.float32, device="cpu")
  assert path is None and isinstance(m, Transformer)
  safetensors_saver.save_lora_merged_model_as_safetensors(None, str(tmp_path), m)
  m2, path = automodel.AutoModel.from_pretrained("Qwen/Qwen3-0.6B", model_path=str(tmp_path), model_config=cfg,
                                                 dtype=torch.float32, device="cpu")
  assert path == str(tmp_path)
  assert torch.equal(m.embedder.input_embedding, m2.embedder.input_embedding)
  with pytest.raises(ValueError):
    automodel.AutoModel.from_pretrained("Qwen/Qwen3-0.6B", model_source=automodel.ModelSource.GCS)
  with pytest.raises(FileNotFoundError):
    automodel.download_model("/nonexistent/dir", None, automodel.ModelSource.INTERNAL)


def test_mapping_config_matches_hf_export(tmp_path):
  """The declarative mapping reproduces the exporter's names and tensors, dense and MoE."""
  from tunix_b200.generate import mappings
  from tunix_b200.models import safetensors_saver
  from tunix_b200.models.transformer import ModelConfig, Transformer
  for moe in (False, True):
    kw = dict(num_experts=4, num_experts_per_tok=2, moe_hidden_dim=16) if moe else {}
    cfg = ModelConfig(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=64, num_heads=4, head_dim=8,
                      num_kv_heads=2, use_qk_norm=True, **kw)
    model = Transformer(cfg).init_weights(seed=0)
    want = safetensors_saver.to_hf_state(model)
    mc = mappings.MappingConfig.build(model=model)
    got = mappings.apply(mc, {n: p.detach() for n, p in model.named_parameters()})
    assert set(got) == set(want)
    for k in want:
      assert torch.equal(got[k], want[k]), k
  again = mappings.MappingConfig.build(mapping_obj={"to_hf_mappings": lambda: {"a": ("b", None)}})
  assert again.to_hf_mappings == {"a": ("b", None)}
  assert mappings.MappingConfig.build(mapping_obj=again) is again
  with pytest.raises(KeyError):
    mappings.apply(again, {"zzz": torch.zeros(1)})


def test_script_utils_datasets(tmp_path):
  import json
  from tunix_b200.utils import script_utils
  recs = [{"question": f"q{i}", "answer": f"blah #### {i}"} for i in range(10)]
  (tmp_path / "train.jsonl").write_text("\n".join(json.dumps(r) for r in recs))
  tr, ev = script_utils.get_train_and_eval_datasets(
      str(tmp_path), "train", seed=1, system_prompt="SYS ", batch_size=2, num_batches=4, train_fraction=0.5,
      num_epochs=2, answer_extractor=lambda s: s.split("####")[1].strip())
  tb, eb = list(tr), list(ev)
  assert len(tb) == 4 and len(eb) == 4            # 2 batches x 2 epochs each
  assert tb[0]["prompts"][0].startswith("SYS q") and tb[0]["answer"][0].isdigit()
  with script_utils.profile_and_capture_log("t", enable_profile=False):
    pass


def test_gemma3_vision_tower_and_multimodal_merge():
  from tunix_b200.models.gemma3 import vision
  from tunix_b200.models.transformer import ModelConfig, Transformer
  torch.manual_seed(0)
  vc = vision.SigLIPConfig(image_height=28, image_width=28, patch_size=(7, 7), width=32, depth=2, mlp_dim=64,
                           num_heads=4, num_mm_tokens_per_image_prepool=16, num_mm_tokens_per_image=4)
  tower = vision.SigLiP(vc)
  imgs = torch.randn(2, 3, 28, 28, 3)
  soft = tower(imgs)
  assert soft.shape == (2, 3, 4, 32) and not soft.requires_grad
  # the exit layer averages 2x2 windows of the 4x4 patch grid
  grid = torch.arange(16.0).view(1, 16, 1)
  assert vision.VisionExit(4)(grid).flatten().tolist() == [2.5, 4.5, 10.5, 12.5]

  cfg = ModelConfig(num_layers=2, vocab_size=256, embed_dim=32, hidden_dim=64, num_heads=4, head_dim=8, num_kv_heads=2)
  mm = vision.Gemma3Multimodal(Transformer(cfg).init_weights(seed=0, scale=0.2), vc)
  with torch.no_grad():
    mm.mm_input_projection.normal_(0, 0.2)
    mm.mm_soft_embedding_norm.w.fill_(1.0)
    mm.vision_encoder.siglip_encoder.pos_embedding.normal_(0, 0.02)
  ph = vc.soft_token_placeholder
  toks = torch.tensor([[5, ph, ph, ph, ph, 9, 10, ph, ph, ph, ph, 11], [7, 8, ph, ph, ph, ph, 12, 13, 14, 15, 16, 17]])
  images = torch.randn(2, 2, 28, 28, 3)
  logits, _ = mm(toks, images=images)
  assert logits.shape == (2, 12, 256) and torch.isfinite(logits).all()
  mask = vision.multimodal_attention_mask(toks, ph, 4)
  assert mask[0, 1, 4] and mask[0, 4, 1]                     # inside one image: both directions
  assert not mask[0, 1, 7] and mask[0, 7, 1]                 # across images: causal only
  assert not mask[0, 0, 1]
  # changing the second image changes only what follows it; the text-only path ignores images
  images2 = images.clone()
  images2[0, 1] += 1.0
  logits2, _ = mm(toks, images=images2)
  assert torch.allclose(logits[0, :7], logits2[0, :7], atol=1e-5) and not torch.allclose(logits[0, 7:], logits2[0, 7:])
  assert torch.allclose(logits[1], logits2[1], atol=1e-5)
  emb = vision.merge_embeddings(torch.zeros(1, 5, 2), torch.arange(8.0).view(1, 2, 2, 2),
                                torch.tensor([[False, True, True, False, True]]))
  assert emb[0].tolist() == [[0, 0], [0, 1], [2, 3], [0, 0], [4, 5]]


def test_oss_download_helpers_fail_clearly_offline(tmp_path, monkeypatch):
  import pytest
  from tunix_b200.oss import utils as oss
  assert oss.pathways_available() is False
  assert oss.load_file_from_gcs(str(tmp_path)) == str(tmp_path)          # local paths pass through
  monkeypatch.setenv("HF_HUB_OFFLINE", "1")
  with pytest.raises(FileNotFoundError, match="local directory"):
    oss.hf_pipeline("some-org/definitely-not-cached-model", str(tmp_path / "dl"))
  with pytest.raises(FileNotFoundError, match="local directory"):
    oss.load_file_from_gcs("gs://no-such-bucket-tunix-b200/ckpt", str(tmp_path / "gcs"))
