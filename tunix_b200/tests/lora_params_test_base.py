"""Base class for tests of LoRA-merged export, one subclass per architecture
(tunix/tests/lora_params_test_base.py:36-300).

A subclass says which architecture (`create_config`) and, when the family needs it, how the file is written
(`save_merged_model`) and read back (`create_model_from_checkpoint`). The base class then checks what must hold for
every family:

  * the exported weight of every adapted projection equals W + (alpha / rank) * B A computed here, independently of
    the framework's merge;
  * projections without adapters are exported unchanged;
  * a model loaded from the exported file computes the same logits as the model with its adapters attached;
  * the export leaves the adapted model as it was (adapters still there, still trainable).

pytest-style: subclasses are plain classes named `Test...`; `tmp_path` is pytest's fixture.
"""
from __future__ import annotations

import os
import re
from typing import Any, Dict, List

import torch

from ..models import lora as lora_lib, safetensors_io, safetensors_saver
from ..models.transformer import ModelConfig, Transformer
from . import test_common


class LoraParamsTestBase:
  rank = 4
  alpha = 16.0
  random_seed = 42
  lora_scale = 0.05
  base_model_scale = 0.3
  atol = 1e-5

  # ---- what a subclass provides ---------------------------------------------------------------
  def create_config(self) -> ModelConfig:
    raise NotImplementedError

  def get_lora_module_path(self) -> str:
    return ".*(q_proj|k_proj|v_proj|o_proj|gate_proj|up_proj|down_proj)"

  def save_merged_model(self, lora_model: torch.nn.Module, output_dir: str) -> str:
    return safetensors_saver.save_lora_merged_model_as_safetensors(None, output_dir, lora_model, rank=self.rank,
                                                                   alpha=self.alpha)

  def create_model_from_checkpoint(self, checkpoint_dir: str) -> torch.nn.Module:
    from ..models import safetensors_loader
    return safetensors_loader.load_and_create_model(checkpoint_dir, Transformer, self.create_config(), None,
                                                    dtype=torch.float32, device="cpu")

  # ---- shared construction ----------------------------------------------------------------------
  def create_base_model(self) -> Transformer:
    return Transformer(self.create_config()).init_weights(seed=self.random_seed, scale=self.base_model_scale)

  def create_lora_model(self) -> Transformer:
    model = lora_lib.apply_lora_to_model(self.create_base_model(), rank=self.rank, alpha=self.alpha,
                                         module_path=self.get_lora_module_path())
    generator = torch.Generator().manual_seed(self.random_seed + 1)
    with torch.no_grad():
      for _, p in model.named_parameters():
        if getattr(p, "is_lora", False):
          p.copy_(torch.randn(p.shape, generator=generator).to(p.dtype) * self.lora_scale)
    return model

  def expected_merged_state(self, lora_model: torch.nn.Module) -> Dict[str, torch.Tensor]:
    """Exported-name -> tensor, with the adapter products added by hand (no call into `merge_lora`)."""
    from ..models.transformer import Linear
    import copy
    plain = copy.deepcopy(lora_model)
    with torch.no_grad():
      for mod in plain.modules():
        if isinstance(mod, Linear) and len(mod.lora_a):
          w = mod.weight().detach().float().clone()
          for key in list(mod.lora_a.keys()):
            lo, hi = mod.slices["" if key == "w" else key]
            w[lo:hi] += (self.alpha / self.rank) * (mod.lora_b[key].float() @ mod.lora_a[key].float())
          mod.quant = None
          mod.w.data = w.to(mod.w.dtype)
          mod.lora_a.clear(); mod.lora_b.clear(); mod.lora_scale.clear()
    return safetensors_saver.to_hf_state(plain)

  def adapted_export_names(self, state: Dict[str, torch.Tensor]) -> List[str]:
    wanted = re.compile(self.get_lora_module_path())
    return [k for k in state if wanted.search(k.rsplit(".weight", 1)[0])]

  # ---- the tests every family gets ------------------------------------------------------------------
  def test_exported_projections_hold_base_plus_scaled_adapter_product(self, tmp_path):
    lora_model = self.create_lora_model()
    out = self.save_merged_model(lora_model, str(tmp_path / "merged"))
    assert os.path.isfile(out)
    written = {name: tensor.clone() for name, tensor in safetensors_io.iter_tensors(out)}
    expected = self.expected_merged_state(lora_model)
    assert sorted(written) == sorted(expected)
    adapted = self.adapted_export_names(expected)
    assert adapted, "the module path matched no exported projection"
    base = safetensors_saver.to_hf_state(self.create_base_model())
    for name in written:
      torch.testing.assert_close(written[name].float(), expected[name].float(), atol=self.atol, rtol=0, msg=name)
      if name in adapted:
        assert not torch.allclose(written[name].float(), base[name].float(), atol=self.atol), f"{name} did not change"
      else:
        torch.testing.assert_close(written[name].float(), base[name].float(), atol=0, rtol=0, msg=name)

  def test_a_model_loaded_from_the_export_matches_the_adapted_model(self, tmp_path):
    lora_model = self.create_lora_model()
    self.save_merged_model(lora_model, str(tmp_path / "merged"))
    loaded = self.create_model_from_checkpoint(str(tmp_path / "merged"))
    inputs = test_common.get_dummy_inputs_for_lora_toy_transformer_tests(vocab_size=self.create_config().vocab_size)
    with torch.no_grad():
      want = lora_model(inputs["input_tokens"], inputs["positions"], None, inputs["attention_mask"])[0]
      got = loaded(inputs["input_tokens"], inputs["positions"], None, inputs["attention_mask"])[0]
    torch.testing.assert_close(got.float(), want.float(), atol=1e-4, rtol=1e-4)

  def test_the_export_leaves_the_adapted_model_untouched(self, tmp_path):
    lora_model = self.create_lora_model()
    before = {n: p.detach().clone() for n, p in lora_model.named_parameters()}
    self.save_merged_model(lora_model, str(tmp_path / "merged"))
    assert lora_lib.is_lora_enabled(lora_model)
    test_common.assert_equal(before, dict(lora_model.named_parameters()))
    assert all(p.requires_grad == bool(getattr(p, "is_lora", False)) for p in lora_model.parameters())
