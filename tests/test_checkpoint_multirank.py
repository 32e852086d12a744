"""Checkpointing of sharded state on 2 gloo ranks: one agreed save decision, per-rank shard files,
expert-parallel weights, and a restore at another job size."""
import os
import subprocess
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(tmp_path, moe: int, port: int, ocdbt: int = 0):
  out, root = str(tmp_path / "res.pt"), str(tmp_path / "ckpt")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_ckpt_worker.py"), "--out", out, "--root", root,
         "--moe", str(moe), "--ocdbt", str(ocdbt)]
  r = subprocess.run(cmd, env=dict(os.environ, OMP_NUM_THREADS="2"), capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  return torch.load(out, weights_only=False), root


def test_ranks_agree_on_saves_and_every_rank_gets_its_own_state_back(tmp_path):
  got, root = _run(tmp_path, 1, 29681)
  r0, r1 = got["ranks"]
  # the run finished (no rank waited alone in a collective) and the forced final save exists
  assert r0["steps"] == r1["steps"] and r0["steps"][-1] == 6
  assert len(r0["steps"]) < 6            # the slow writer made rank 0 skip steps, and rank 1 followed it
  for r in (r0, r1):
    assert r["restored_step"] == 6 and r["count"] == r["count_saved"] == 6
    assert r["param_err"] == 0.0 and r["mu_err"] == 0.0 and r["master_err"] == 0.0 and r["local_err"] == 0.0
  assert max(r0["mu_norm"], r1["mu_norm"]) > 0       # (a rank's slices of this tiny model may be all padding)
  assert r0["expert_sig"] != r1["expert_sig"]       # each rank restored its own experts, not rank 0's
  # on disk: one chunk file per rank for the flat state and for the expert arrays, no temporary directory left
  step_dir = os.path.join(root, "6")
  assert sorted(f for f in os.listdir(os.path.join(step_dir, "optimizer_state", "mu.flat.value")) if f[0] != ".") == ["0", "1"]
  experts = os.path.join(step_dir, "model_params", "layers.0.mlp.down_proj.value")
  assert sorted(f for f in os.listdir(experts) if f[0] != ".") == ["0.0.0", "1.0.0"]
  assert not [d for d in os.listdir(root) if ".tmp-" in d]


def test_flat_state_restores_at_another_job_size(tmp_path):
  """Saved by 2 ranks, read back by a single process: its one shard is the whole flat range."""
  got, root = _run(tmp_path, 0, 29682)
  from tunix_b200 import optim
  from tunix_b200.common.configs import TrainingConfig
  from tunix_b200.sft.peft_trainer import PeftTrainer
  sys.path.insert(0, HERE)
  import _ckpt_worker
  model = _ckpt_worker.build(None, False)
  tc = TrainingConfig(eval_every_n_steps=100, pbar_description=None, checkpoint_root_directory=root)
  tr = PeftTrainer(model, optim.adamw(5e-3, weight_decay=0.01), tc)
  assert tr.train_steps == 6
  mu = tr.optimizer.opt_state["mu"]["flat"]
  n = got["index"]["used"]
  assert float((mu[:n] - got["full_mu"][:n]).abs().max()) == 0.0
  tr.checkpoint_manager.close()


def test_per_process_key_value_stores_hold_the_same_checkpoint(tmp_path):
  """With `use_ocdbt` every rank writes one store `ocdbt.process_<r>` per item instead of a file per array chunk;
  the restore reads the union of the stores and every rank still gets its own shards back."""
  got, root = _run(tmp_path, 1, 29683, ocdbt=1)
  for r in got["ranks"]:
    assert r["restored_step"] == 6 and r["param_err"] == 0.0 and r["mu_err"] == 0.0 and r["local_err"] == 0.0
  assert got["ranks"][0]["expert_sig"] != got["ranks"][1]["expert_sig"]
  item = os.path.join(root, "6", "optimizer_state")
  names = sorted(os.listdir(item))
  assert "ocdbt.process_0" in names and "ocdbt.process_1" in names and "mu.flat.value" not in names
  assert sorted(os.listdir(os.path.join(item, "ocdbt.process_1"))) == ["d", "manifest.ocdbt"]
  from tunix_b200.ckpt import orbax_layout
  kv = orbax_layout.open_kv(item)
  assert kv.get("mu.flat.value/.zarray") is not None and kv.get("mu.flat.value/0") and kv.get("mu.flat.value/1")
