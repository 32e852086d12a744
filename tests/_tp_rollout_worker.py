"""Worker for the tensor-parallel rollout test (2 GPUs): the trainer's flat store is re-sharded into each
rank's tensor-parallel slice by the copy kernel (own replica and a peer's replica as the source), the
paged engine decodes on it with the in-kernel all-reduce exits, and the result is compared with the
unsharded engine."""
import argparse
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--out", required=True)
  a = ap.parse_args()
  import torch.distributed as dist
  from tunix_b200.dist import fsdp, mesh as mesh_lib, weight_sync
  from tunix_b200.models.transformer import ModelConfig, Transformer
  from tunix_b200.ops import _lib
  from tunix_b200.rollout import EngineConfig, PagedEngine
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  dev = torch.device("cuda", local)
  mesh_lib.init_distributed("nccl", timeout_s=120)
  world, rank = dist.get_world_size(), dist.get_rank()
  fs_mesh = mesh_lib.create_mesh((world,), ("fsdp",))
  tp_mesh = mesh_lib.create_mesh((1, world), ("dp", "tp"))
  cfg = ModelConfig(num_layers=2, vocab_size=512, embed_dim=512, hidden_dim=1024, num_heads=8, head_dim=128,
                    num_kv_heads=2, use_qk_norm=True, dtype=torch.bfloat16, max_position=256)
  trainer = fsdp.shard_model(Transformer(cfg, device=dev).init_weights(seed=0, scale=0.05), fs_mesh)
  res = {"rank": rank}
  rng = np.random.default_rng(0)
  prompts = [rng.integers(3, 500, size=n).tolist() for n in (5, 37, 64, 20)]
  trainer.eval()

  def reference_logprobs(prompt, toks):
    """Log-probs of `toks` after `prompt` from a plain forward of the unsharded model."""
    seq = torch.tensor([prompt + list(toks)], device=dev)
    with torch.no_grad():
      logits, _ = trainer(seq, None, None, None)
    lp = torch.log_softmax(logits[0, len(prompt) - 1:-1].float(), -1)
    return lp.gather(-1, seq[0, len(prompt):, None])[:, 0].cpu().numpy()

  for source in (rank, (rank + 1) % world):          # own replica, then the peer's over NVLink
    rep = weight_sync.RolloutReplica(trainer, tp_mesh, "tp", source_rank=source, double_buffer=(source != rank))
    v = rep.sync()
    assert rep.completed_version() == v
    # the slice equals what slicing the full model gives
    from tunix_b200.dist import tp as tp_lib
    ref = tp_lib.shard_model_tp(trainer, tp_mesh)
    worst = 0.0
    rp = dict(rep.model.named_parameters())
    for n, p in ref.named_parameters():
      q = rp[n]
      worst = max(worst, float((p.float() - q.float()).abs().max()))
    res[f"slice_err_{'own' if source == rank else 'peer'}"] = worst
    res[f"sync_ms_{'own' if source == rank else 'peer'}"] = rep.sync_ms()
    res[f"bytes_{'own' if source == rank else 'peer'}"] = rep.plan.bytes
    for graphs in (False, True):
      eng = PagedEngine(rep.model, EngineConfig(page_size=16, max_batch=8, max_seq_len=128, use_cuda_graphs=graphs))
      got = eng.generate(prompts, 16, temperature=1.0, seed=3)
      key = f"{'own' if source == rank else 'peer'}_{'graph' if graphs else 'eager'}"
      # both ranks of the group sampled the same tokens, and their log-probs are the unsharded model's
      toks = torch.tensor([t.tolist() for t in got.tokens], device=dev)
      peer_toks = [torch.empty_like(toks) for _ in range(world)]
      dist.all_gather(peer_toks, toks)
      res[f"same_tokens_{key}"] = all(torch.equal(peer_toks[0], t) for t in peer_toks)
      res[f"lp_err_{key}"] = max(float(np.abs(lp - reference_logprobs(p, t)).max())
                                 for p, t, lp in zip(prompts, got.tokens, got.logprobs))
      res[f"captured_{key}"] = bool(graphs and any(v is not False for v in eng._graphs.values()))
    del rep, eng, ref
  # 96 sequences: above 64 rows the tensor-parallel exits run as two chunks of the skinny kernel and the plain
  # products take the general GEMM; tokens still agree across the group and with the unsharded model
  rep = weight_sync.RolloutReplica(trainer, tp_mesh, "tp")
  rep.sync()
  many = [rng.integers(3, 500, size=int(n)).tolist() for n in rng.integers(4, 40, size=96)]
  eng = PagedEngine(rep.model, EngineConfig(page_size=16, max_batch=96, max_seq_len=128, use_cuda_graphs=True))
  got = eng.generate(many, 8, temperature=1.0, seed=5)
  toks = torch.tensor([t.tolist() for t in got.tokens], device=dev)
  peer_toks = [torch.empty_like(toks) for _ in range(world)]
  dist.all_gather(peer_toks, toks)
  res["same_tokens_96"] = all(torch.equal(peer_toks[0], t) for t in peer_toks)
  res["lp_err_96"] = max(float(np.abs(lp - reference_logprobs(p, t)).max())
                         for p, t, lp in list(zip(many, got.tokens, got.logprobs))[::9])
  del rep, eng
  # a weight change reaches the replica through the next sync
  rep = weight_sync.RolloutReplica(trainer, tp_mesh, "tp")
  rep.sync()
  before = next(iter(rep.model.parameters())).float().sum().item()
  with torch.no_grad():
    trainer.flat_store.flat_param.mul_(1.5)
  rep.sync()
  after = next(iter(rep.model.parameters())).float().sum().item()
  res["update_ratio"] = after / before
  torch.cuda.synchronize()
  _lib.check_status()
  allres = [None] * world
  dist.all_gather_object(allres, res)
  if rank == 0:
    torch.save(allres, a.out)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
