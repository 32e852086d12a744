"""Worker for the multi-rank FSDP tests (launched under torchrun).

Trains a tiny decoder for a few optimizer steps with the flat sharded store and writes the final
parameters of rank 0 to `--out`. With WORLD_SIZE=1 it produces the unsharded reference run."""
import argparse
import contextlib
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--out", required=True)
  ap.add_argument("--transport", default="nccl")
  ap.add_argument("--device", default="cuda")
  ap.add_argument("--steps", type=int, default=3)
  ap.add_argument("--mode", default="")           # resident | sharded; "" = resident on CUDA, no store on CPU
  ap.add_argument("--layers", type=int, default=2)
  ap.add_argument("--remat", type=int, default=0)
  a = ap.parse_args()
  from tunix_b200 import optim
  from tunix_b200.common.configs import TrainingConfig
  from tunix_b200.dist import fsdp, mesh as mesh_lib
  from tunix_b200.models.llama3.model import ModelConfig
  from tunix_b200.models.transformer import Transformer
  from tunix_b200.ops import _lib
  from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput

  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  cuda = a.device == "cuda"
  mesh = None
  if world > 1:
    mesh_lib.init_distributed("nccl" if cuda else "gloo", timeout_s=120)
    mesh = mesh_lib.create_mesh((world,), ("fsdp",))
    mesh_lib.set_current_mesh(mesh)
  dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0"))) if cuda else torch.device("cpu")
  if cuda:
    torch.cuda.set_device(dev)
  from tunix_b200.models.transformer import RematConfig
  cfg = ModelConfig(num_layers=a.layers, remat_config=RematConfig.BLOCK if a.remat else RematConfig.NONE, vocab_size=512, embed_dim=256, hidden_dim=512, num_heads=4, head_dim=64,
                    num_kv_heads=2, dtype=torch.bfloat16 if cuda else torch.float32, max_position=64)
  model = Transformer(cfg, device=dev).init_weights(seed=0)
  if cuda or a.mode:
    model = fsdp.shard_model(model, mesh, transport=a.transport, mode=a.mode or None)
  tc = TrainingConfig(eval_every_n_steps=100, gradient_accumulation_steps=2, max_grad_norm=1.0, pbar_description=None)
  tr = PeftTrainer(model, optim.adamw(2e-3, weight_decay=0.01), tc)
  tr.with_grad_sync(fsdp.GradSync(model, mesh))
  g = torch.Generator().manual_seed(7)
  data = []
  for _ in range(a.steps * 2):
    tok = torch.randint(0, 512, (4, 64), generator=g)     # global batch; every rank slices its share
    mask = torch.ones(4, 64)
    mask[:, : int(torch.randint(0, 32, (1,), generator=g))] = 0
    data.append(TrainingInput(tok, mask))
  tr.train(data)
  if cuda:
    torch.cuda.synchronize()
    _lib.check_status()
  store = getattr(model, "flat_store", None)
  with (store.summon_full_params() if store is not None else contextlib.nullcontext()):
    params = {n: p.detach().float().cpu() for n, p in model.named_parameters()}
  if rank == 0:
    torch.save({"params": params, "loss": tr.metrics_logger.get_metric_history("", "loss", "train"),
                "memory": store.memory_report() if hasattr(store, "memory_report") else None}, a.out)
  if world > 1:
    torch.distributed.barrier()
    torch.distributed.destroy_process_group()


if __name__ == "__main__":
  main()
