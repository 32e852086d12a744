"""Compares this framework's forward pass with Hugging Face transformers on the same weights.

  python examples/tools/forward_pass_logit_checker.py --self-test                       # tiny random Llama, no files
  python examples/tools/forward_pass_logit_checker.py --checkpoint /path/to/hf_dir --model llama3.2-1b \\
      --prompt "The capital of France is" --dtype bfloat16

With `--checkpoint`, the directory is loaded twice: by `transformers.AutoModelForCausalLM` and by this framework's
`create_model_from_safe_tensors`; both run the same token ids and the script reports the largest absolute logit
difference, the KL divergence of the next-token distributions, whether the arg-max tokens agree at every position,
and each side's top-5 next tokens. Exit code 1 when the difference exceeds `--atol` (relative to the logit range).
`--self-test` builds a two-layer random Llama in memory instead, which checks the tool and the name mapping without
any checkpoint on disk.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

import torch
import torch.nn.functional as F


def compare(ours: torch.nn.Module, theirs: torch.nn.Module, tokens: torch.Tensor, top: int = 5) -> dict:
  positions = torch.arange(tokens.shape[1], device=tokens.device)[None].expand_as(tokens)
  with torch.no_grad():
    got = ours(tokens, positions, None, None)[0].float()
    want = theirs(tokens).logits.float()
  diff = (got - want).abs()
  log_p, log_q = F.log_softmax(want, -1), F.log_softmax(got, -1)
  return {"max_abs_diff": diff.max().item(), "mean_abs_diff": diff.mean().item(), "logit_range": want.abs().max().item(),
          "kl": (log_p.exp() * (log_p - log_q)).sum(-1).mean().item(),
          "argmax_agreement": (got.argmax(-1) == want.argmax(-1)).float().mean().item(),
          "top_ours": got[0, -1].topk(top).indices.tolist(), "top_theirs": want[0, -1].topk(top).indices.tolist()}


def self_test_models():
  from transformers import LlamaConfig, LlamaForCausalLM
  from tunix_b200.models import safetensors_loader
  from tunix_b200.models.llama3 import model as llama
  from tunix_b200.models.transformer import Transformer
  torch.manual_seed(0)
  hf_cfg = LlamaConfig(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, vocab_size=128, max_position_embeddings=64, rms_norm_eps=1e-6,
                       rope_theta=500000.0, tie_word_embeddings=False, attention_dropout=0.0)
  theirs = LlamaForCausalLM(hf_cfg).eval().float()
  cfg = llama.ModelConfig(num_layers=2, vocab_size=128, embed_dim=64, hidden_dim=96, num_heads=4, head_dim=16,
                          num_kv_heads=2, norm_eps=1e-6, dtype=torch.float32, max_position=64,
                          rope_theta=500000.0, weight_tying=False)
  ours = Transformer(cfg)
  state, _ = safetensors_loader.convert_state(theirs.state_dict().items(), gemma_norms=False)
  with torch.no_grad():
    for name, p in ours.named_parameters():
      p.copy_(state[name])
  return ours, theirs, torch.randint(0, 128, (2, 24))


def checkpoint_models(args):
  from transformers import AutoModelForCausalLM, AutoTokenizer
  from tunix_b200.models import automodel
  dtype = getattr(torch, args.dtype)
  device = "cuda" if torch.cuda.is_available() else "cpu"
  theirs = AutoModelForCausalLM.from_pretrained(args.checkpoint, torch_dtype=dtype).to(device).eval()
  ours = automodel.create_model_from_safe_tensors(args.model, args.checkpoint, dtype=dtype, device=device)
  tokens = AutoTokenizer.from_pretrained(args.checkpoint)(args.prompt, return_tensors="pt").input_ids.to(device)
  return ours, theirs, tokens


def main() -> int:
  ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
  ap.add_argument("--self-test", action="store_true")
  ap.add_argument("--checkpoint", default=None)
  ap.add_argument("--model", default=None, help="preset name of this framework, e.g. llama3.2-1b, qwen3-8b")
  ap.add_argument("--prompt", default="The capital of France is")
  ap.add_argument("--dtype", default="float32", choices=("float32", "bfloat16", "float16"))
  ap.add_argument("--atol", type=float, default=None, help="default 2e-4 in float32, 5e-2 otherwise")
  args = ap.parse_args()
  if not args.self_test and not (args.checkpoint and args.model):
    ap.error("give --self-test, or --checkpoint together with --model")
  ours, theirs, tokens = self_test_models() if args.self_test else checkpoint_models(args)
  report = compare(ours, theirs, tokens)
  for key, value in report.items():
    print(f"{key:18s} {value:.6g}" if isinstance(value, float) else f"{key:18s} {value}")
  atol = args.atol if args.atol is not None else (2e-4 if args.dtype == "float32" else 5e-2)
  ok = report["max_abs_diff"] <= atol * max(1.0, report["logit_range"])
  print("PASS" if ok else f"FAIL: max_abs_diff above {atol} x logit range")
  return 0 if ok else 1


if __name__ == "__main__":
  sys.exit(main())
