"""Worker for the multi-rank checkpoint test: 2 gloo ranks, a tiny MoE decoder with experts split over
the ranks and a flat sharded optimizer state; saves under a time-based policy with a slow writer on
rank 0, restores into fresh objects, and reports what each rank got back."""
import argparse
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def build(mesh, moe: bool):
  from tunix_b200.dist import fsdp, moe as dist_moe
  from tunix_b200.models.transformer import ModelConfig, Transformer
  cfg = ModelConfig(num_layers=2, vocab_size=64, embed_dim=32, hidden_dim=48, num_heads=4, head_dim=8, num_kv_heads=2,
                    **(dict(num_experts=4, num_experts_per_tok=2, moe_hidden_dim=24) if moe else {}))
  model = Transformer(cfg).init_weights(seed=0, scale=0.3)
  if moe and mesh is not None:
    dist_moe.shard_experts(model, mesh)
  return fsdp.shard_model(model, mesh, transport="nccl")


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--out", required=True)
  ap.add_argument("--root", required=True)
  ap.add_argument("--moe", type=int, default=1)
  ap.add_argument("--ocdbt", type=int, default=0)
  a = ap.parse_args()
  import torch.distributed as dist
  from tunix_b200 import optim
  from tunix_b200.common.configs import TrainingConfig
  from tunix_b200.dist import fsdp, mesh as mesh_lib
  from tunix_b200.sft import checkpoint_manager as cm, checkpoint_options as co
  from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput
  mesh_lib.init_distributed("gloo", timeout_s=120)
  world, rank = dist.get_world_size(), dist.get_rank()
  mesh = mesh_lib.create_mesh((world,), ("fsdp",))
  mesh_lib.set_current_mesh(mesh)
  opts = co.TunixCheckpointingOptions(save_decision_policy=co.ContinuousCheckpointingPolicy(minimum_interval_secs=0.25),
                                      preservation_policy=co.LatestN(n=10), enable_async_checkpointing=True,
                                      async_options=co.AsyncOptions(timeout_secs=60), use_ocdbt=bool(a.ocdbt))
  tc = TrainingConfig(eval_every_n_steps=100, max_grad_norm=1.0, pbar_description=None, data_sharding_axis=(),
                      checkpoint_root_directory=a.root, checkpointing_options=opts)

  def trainer():
    model = build(mesh, bool(a.moe))
    tr = PeftTrainer(model, optim.adamw(5e-3, weight_decay=0.01), tc)
    tr.with_grad_sync(fsdp.GradSync(model, mesh))
    return model, tr

  model, tr = trainer()
  if rank == 0:
    # rank 0's writer is slow and rank 1's clock runs ahead: alone, the ranks would disagree on most steps
    orig = tr.checkpoint_manager._write

    def slow(*args, **kw):
      time.sleep(0.4)
      return orig(*args, **kw)
    tr.checkpoint_manager._write = slow
  else:
    tr.checkpoint_manager._last_save_time = time.time() - 100.0
  g = torch.Generator().manual_seed(7 + rank)
  data = [TrainingInput(torch.randint(0, 64, (2, 16), generator=g), torch.ones(2, 16)) for _ in range(6)]
  tr.is_managed_externally = True
  for i, b in enumerate(data):
    tr.train([b])
    time.sleep(0.1)
  tr.close()
  dist.barrier()
  steps = cm.orbax_layout.list_steps(a.root)
  saved = {n: p.detach().clone() for n, p in model.named_parameters()}
  st = tr.optimizer.opt_state
  saved_mu = st["mu"]["flat"].clone()
  saved_local = st["mu"]["local"].clone() if "local" in st["mu"] else None
  count = int(st["count"])
  # ---- restore into fresh objects
  model2, tr2 = trainer()
  res = {"rank": rank, "steps": steps, "restored_step": tr2.train_steps, "count": int(tr2.optimizer.opt_state["count"]),
         "count_saved": count}
  res["param_err"] = max(float((p.detach() - saved[n]).abs().max()) for n, p in model2.named_parameters())
  st2 = tr2.optimizer.opt_state
  res["mu_err"] = float((st2["mu"]["flat"] - saved_mu).abs().max())
  res["master_err"] = float((st2["master"]["flat"] - st["master"]["flat"]).abs().max())
  if saved_local is not None:
    res["local_err"] = float((st2["mu"]["local"] - saved_local).abs().max())
    e = [p for n, p in model2.named_parameters() if n.endswith("mlp.down_proj")][0]
    res["expert_sig"] = float(e.detach().double().sum())
  res["mu_norm"] = float(saved_mu.norm())
  full_mu = model.flat_store.full_state_tensor(st["mu"]["flat"])
  allres = [None] * world
  dist.all_gather_object(allres, res)
  if rank == 0:
    torch.save({"ranks": allres, "full_mu": full_mu, "index": model.flat_store.flat_index()}, a.out)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
