"""Supervised / LoRA fine-tuning entry point (tunix/cli/peft_main.py:35-112).

  python -m tunix_b200.cli.peft_main base_config.yaml model_config.model_source=dummy dataset_name=synthetic ...
  torchrun --nproc-per-node 8 -m tunix_b200.cli.peft_main base_config.yaml model_config.mesh.shape="(8,1)" ...
"""
from __future__ import annotations

import logging
import sys

import torch

from ..dist import mesh as dist_mesh
from ..examples.data import translation_dataset as data_lib
from ..sft import peft_trainer, utils as sft_utils
from ..utils import mesh as mesh_lib
from . import config
from .utils import model as model_lib


class PeftPipeline(config.HyperParameters):
  def run_peft_trainer(self):
    shape, names = self.parse_mesh_config("model_config")
    n = 1
    for s in shape:
      n *= s
    if n > 1:
      dist_mesh.init_distributed()
    mesh = mesh_lib.create_mesh(shape, names)
    model, tokenizer_path = model_lib.create_model(self.config["model_config"], self.config["tokenizer_config"], mesh)
    tokenizer = model_lib.create_tokenizer(self.config["tokenizer_config"], tokenizer_path)
    optimizer = self.create_optimizer("optimizer_config")
    trainer = peft_trainer.PeftTrainer(
        model, optimizer, peft_trainer.TrainingConfig(**self.obtain_training_config_dict("training_config")))
    pad = tokenizer.pad_id() or 0

    def gen_model_input_fn(x: peft_trainer.TrainingInput):
      tokens = torch.as_tensor(x.input_tokens)
      pad_mask = tokens != pad
      return {"input_tokens": tokens, "input_mask": torch.as_tensor(x.input_mask),
              "positions": sft_utils.build_positions_from_mask(pad_mask),
              "attention_mask": sft_utils.make_causal_attn_mask(pad_mask)}
    trainer = trainer.with_gen_model_input_fn(gen_model_input_fn)
    train_ds, eval_ds = data_lib.create_datasets(
        dataset_name=self.config["dataset_name"], global_batch_size=self.config["batch_size"],
        max_target_length=self.config["max_target_length"], num_train_epochs=self.config["num_train_epochs"],
        tokenizer=tokenizer, tfds_download=self.config["tfds_download"])
    with mesh:
      trainer.train(train_ds, eval_ds)
    trainer.close()
    return trainer


def main(argv, **kwargs):
  pipeline = PeftPipeline(argv, **kwargs)
  logging.info("--- Launching PEFT pipeline with following config ---\n%r\n--------------------------", pipeline.config)
  return pipeline.run_peft_trainer()


if __name__ == "__main__":
  logging.basicConfig(level=logging.INFO)
  main(sys.argv)
