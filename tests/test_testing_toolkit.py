"""The testing toolkit shipped in the package: tree comparisons, toy models, the fixed-vocabulary tokenizer, output
validation, and the LoRA export base class run for two architectures."""
import numpy as np
import pytest
import torch

from tunix_b200.rl import common as rl_common
from tunix_b200.tests import lora_params_test_base, test_common as tc
from tunix_b200.utils import torch_utils


def test_tree_comparisons_name_the_leaf_that_differs():
  a = {"layers": [{"w": torch.ones(2, 2), "b": np.zeros(2)}, {"w": torch.zeros(1)}], "step": 3, "none": None}
  b = {"layers": [{"w": torch.ones(2, 2), "b": np.zeros(2)}, {"w": torch.zeros(1)}], "step": 3, "none": None}
  tc.assert_equal(a, b)
  tc.assert_close(a, b)
  b["layers"][0]["w"] = torch.ones(2, 2) + 1e-7
  tc.assert_close(a, b)
  with pytest.raises(AssertionError, match=r"layers\[0\]/w"):
    tc.assert_equal(a, b)
  with pytest.raises(AssertionError, match=r"layers\[0\]/b is equal"):
    tc.assert_not_equal(a, b)
  tc.assert_not_equal({"w": torch.zeros(2)}, {"w": torch.ones(2)})
  with pytest.raises(AssertionError, match="structure"):
    tc.assert_equal({"w": 1}, {"v": 1})
  m1, m2 = tc.ToyTransformer(seed=1), tc.ToyTransformer(seed=1)
  tc.assert_equal(m1, m2)                               # modules compare by state dict
  tc.assert_not_equal({"e": m1.state_dict()[next(iter(m1.state_dict()))]},
                      {"e": tc.ToyTransformer(seed=2).state_dict()[next(iter(m1.state_dict()))]})


def test_toy_models_run_through_the_framework_paths():
  model = tc.ToyTransformer(num_layers=2)
  assert model.config.num_layers == 2 and model.config.vocab_size == 256
  inputs = tc.get_dummy_inputs_for_lora_toy_transformer_tests()
  logits, _ = model(inputs["input_tokens"], inputs["positions"], None, inputs["attention_mask"])
  assert logits.shape == (2, 8, 256)
  scorer = tc.ToyTransformerWithScoreHead(model)
  scores, _ = scorer(inputs["input_tokens"], inputs["positions"], None, inputs["attention_mask"])
  assert scores.shape == (2, 8, 1)
  per_token = rl_common.compute_score(scorer, inputs["input_tokens"][:, :3], inputs["input_tokens"][:, 3:], 0, 2)
  assert per_token.shape == (2, 8)
  lora = tc.get_lora_model(tc.ToyTransformer(num_layers=2))
  trainable = [n for n, p in lora.named_parameters() if p.requires_grad]
  assert trainable and all("lora" in n for n in trainable)
  with torch.no_grad():
    changed, _ = lora(inputs["input_tokens"], inputs["positions"], None, inputs["attention_mask"])
  assert not torch.allclose(changed, logits)              # B factors were filled, so the adapters act
  quiet = tc.get_lora_model(tc.ToyTransformer(num_layers=2), randomize_b=False)
  with torch.no_grad():
    same, _ = quiet(inputs["input_tokens"], inputs["positions"], None, inputs["attention_mask"])
  torch.testing.assert_close(same, logits)


def test_the_fixed_vocabulary_tokenizer_speaks_both_dialects():
  v = tc.MockVocab()
  ids = v.encode("Hello world ! unknownword")
  assert ids == [7, 6, 9] and v.decode(ids) == "Hello world !" and v.EncodeAsIds("hello") == [5] and v.DecodeIds([14]) == "Tunix"
  assert (v.pad_id(), v.bos_id(), v.eos_id()) == (0, 1, 2) and v.GetPieceSize() == v.vocab_size() == 22
  assert tc.MockVocab(is_multimodal=True).encode("<img>") == [22] and tc.MockVocab().encode("<img>") == []
  assert tc.MockVocab({"a": 0, "b": 1}).encode("b a b") == [1, 0, 1]


def test_output_validation_and_housekeeping(tmp_path):
  tc.validate_llm_outputs([("capital of France?", ["paris"]), ("2+2", ["4", "four"])], ["It is Paris.", "4, i.e. Four"])
  with pytest.raises(AssertionError, match="does not contain expected keyword"):
    tc.validate_llm_outputs([("capital of France?", ["paris"])], ["Lyon"])
  with pytest.raises(AssertionError, match="1 expectations for 2 outputs"):
    tc.validate_llm_outputs([("q", ["a"])], ["a", "b"])

  class Chat:
    def apply_chat_template(self, messages, tokenize, add_generation_prompt):
      return f"<user>{messages[0]['content']}</user>" + ("<assistant>" if add_generation_prompt else "")
  assert tc.batch_templatize(["hi", "yo"], Chat()) == ["<user>hi</user><assistant>", "<user>yo</user><assistant>"]
  with pytest.raises(TypeError, match="apply_chat_template"):
    tc.batch_templatize(["hi"], object())
  d = tmp_path / "scratch" / "deep"
  d.mkdir(parents=True)
  (d / "f").write_text("x")
  tc.delete_directory(str(tmp_path / "scratch"))
  tc.delete_directory(str(tmp_path / "scratch"))            # absent: nothing to do
  assert not (tmp_path / "scratch").exists()
  tc.free_device_memory()


def test_checkpoint_keys_map_through_exactly_one_pattern():
  mapping = {r"model\.layers\.(\d+)\.self_attn\.q_proj\.weight": (r"layers.\1.attn.q_proj.w", None),
             r"model\.embed_tokens\.weight": ("embedder.input_embedding", (1, 0))}
  assert torch_utils.map_checkpoint_key(mapping, "model.layers.12.self_attn.q_proj.weight") == ("layers.12.attn.q_proj.w", None)
  assert torch_utils.torch_key_to_jax_key(mapping, "model.embed_tokens.weight") == ("embedder.input_embedding", (1, 0))
  with pytest.raises(ValueError, match="no pattern"):
    torch_utils.map_checkpoint_key(mapping, "lm_head.weight")
  mapping[r"model\.embed.*"] = ("other", None)
  with pytest.raises(ValueError, match="2 patterns"):
    torch_utils.map_checkpoint_key(mapping, "model.embed_tokens.weight")


class TestLlamaStyleExport(lora_params_test_base.LoraParamsTestBase):
  def create_config(self):
    return tc.toy_config(vocab_size=64, num_layers=2)


class TestAttentionOnlyExportWithSharedEmbeddings(lora_params_test_base.LoraParamsTestBase):
  rank, alpha = 2, 4.0

  def create_config(self):
    return tc.toy_config(vocab_size=64, num_layers=2, num_kv_heads=4)

  def get_lora_module_path(self):
    return ".*(q_proj|v_proj)"
