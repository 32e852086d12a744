"""Supervised / LoRA fine-tuning entry point (tunix/cli/peft_main.py:35-112).

  python -m tunix_b200.cli.peft_main base_config.yaml model_config.model_source=dummy dataset_name=synthetic ...
  torchrun --nproc-per-node 8 -m tunix_b200.cli.peft_main base_config.yaml model_config.mesh.shape="(8,1)" ...
"""
from __future__ import annotations

import logging
import math
import sys

import torch

from ..dist import mesh as dist_mesh
from ..examples.data import translation_dataset as data_lib
from ..sft import peft_trainer, utils as sft_utils
from ..utils import mesh as mesh_lib
from . import config
from .utils import model as model_lib


def _padding_aware_inputs(pad_id: int):
  """The trainer's input function for right-padded token rows: positions count real tokens only and the causal
  mask hides the padding."""
  def build(example: peft_trainer.TrainingInput):
    tokens = torch.as_tensor(example.input_tokens)
    real = tokens != pad_id
    return dict(input_tokens=tokens, input_mask=torch.as_tensor(example.input_mask),
                positions=sft_utils.build_positions_from_mask(real),
                attention_mask=sft_utils.make_causal_attn_mask(real))
  return build


class PeftPipeline(config.HyperParameters):
  """The stages of the run are methods, so that a recipe can replace one (another dataset, another trainer)."""

  def build_mesh(self):
    shape, names = self.parse_mesh_config("model_config")
    if math.prod(shape) > 1:
      dist_mesh.init_distributed()
    return mesh_lib.create_mesh(shape, names)

  def build_model_and_tokenizer(self, mesh):
    model_cfg, tok_cfg = self.config["model_config"], self.config["tokenizer_config"]
    model, tokenizer_path = model_lib.create_model(model_cfg, tok_cfg, mesh)
    return model, model_lib.create_tokenizer(tok_cfg, tokenizer_path)

  def build_trainer(self, model, tokenizer):
    training = peft_trainer.TrainingConfig(**self.obtain_training_config_dict("training_config"))
    trainer = peft_trainer.PeftTrainer(model, self.create_optimizer("optimizer_config"), training)
    return trainer.with_gen_model_input_fn(_padding_aware_inputs(tokenizer.pad_id() or 0))

  def build_datasets(self, tokenizer):
    keys = ("dataset_name", "max_target_length", "num_train_epochs", "tfds_download")
    return data_lib.create_datasets(global_batch_size=self.config["batch_size"], tokenizer=tokenizer,
                                    **{k: self.config[k] for k in keys})

  def run_peft_trainer(self):
    mesh = self.build_mesh()
    model, tokenizer = self.build_model_and_tokenizer(mesh)
    trainer = self.build_trainer(model, tokenizer)
    train_ds, eval_ds = self.build_datasets(tokenizer)
    try:
      with mesh:
        trainer.train(train_ds, eval_ds)
    finally:
      trainer.close()
    return trainer


def main(argv, **kwargs):
  pipeline = PeftPipeline(argv, **kwargs)
  logging.info("--- Launching PEFT pipeline with following config ---\n%r\n--------------------------", pipeline.config)
  return pipeline.run_peft_trainer()


if __name__ == "__main__":
  logging.basicConfig(level=logging.INFO)
  main(sys.argv)
