"""Save a model as Hugging Face safetensors and load it back through `AutoModel`.

  python examples/model_load/from_safetensors.py                       # tiny random Llama-style model
  python examples/model_load/from_safetensors.py --dir /path/to/Llama-3.2-1B --model-name llama3.2-1b

With `--dir` an existing local checkpoint directory is loaded and one forward pass is run; without it a tiny model
is exported with the saver (fused projections split into q/k/v and gate/up, checkpoint names), loaded back, and the
logits of both are compared.
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch

from tunix_b200.models import automodel, safetensors_io, safetensors_saver
from tunix_b200.models.transformer import ModelConfig, Transformer


def main() -> None:
  ap = argparse.ArgumentParser()
  ap.add_argument("--dir", default="")
  ap.add_argument("--model-name", default="llama3.2-1b")
  args = ap.parse_args()
  dev = "cuda" if torch.cuda.is_available() else "cpu"
  tokens = torch.randint(3, 100, (2, 12), device=dev)
  positions = torch.arange(12, device=dev)[None].expand(2, 12)
  if args.dir:
    model = automodel.create_model_from_safe_tensors(args.model_name, args.dir, dtype=torch.bfloat16, device=dev)
    logits, _ = model(tokens, positions, None, None)
    print("loaded", args.model_name, "logits", tuple(logits.shape))
    return
  cfg = ModelConfig(num_layers=2, vocab_size=128, embed_dim=64, hidden_dim=128, num_heads=4, head_dim=16, num_kv_heads=2)
  model = Transformer(cfg).init_weights(seed=0, scale=0.1).to(dev)
  with tempfile.TemporaryDirectory() as d:
    safetensors_io.save_file(safetensors_saver.to_hf_state(model), os.path.join(d, "model.safetensors"))
    again = automodel.create_model_from_safe_tensors("custom", d, model_config=cfg, dtype=torch.float32, device=dev)
  with torch.no_grad():
    a, _ = model(tokens, positions, None, None)
    b, _ = again(tokens, positions, None, None)
  print("max |logit difference| after the round trip:", float((a - b).abs().max()))


if __name__ == "__main__":
  main()
