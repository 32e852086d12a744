"""Two gloo ranks on CPU run GRPO through RLCluster with a sharded actor and a shared-storage rollout."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def test_grpo_two_ranks_cpu(tmp_path):
  out = str(tmp_path / "dp.pt")
  env = dict(os.environ, OMP_NUM_THREADS="2")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", "29641", os.path.join(HERE, "_grpo_dp_worker.py"), "--out", out]
  r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  got = torch.load(out, weights_only=False)
  assert got["steps"] == 2
  assert got["moved"] > 0                                   # the actor was trained
  assert abs(got["checksums"][0] - got["checksums"][1]) < 1e-6 * max(1.0, abs(got["checksums"][0]))
  assert all(l == l for l in got["loss"])                   # no NaN


def test_moe_expert_parallel_two_ranks_cpu(tmp_path):
  """Dispatch / grouped MLP / combine over 2 ranks equals the single-rank layer, forward and backward."""
  out = str(tmp_path / "ep.pt")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", "29651", os.path.join(HERE, "_moe_ep_worker.py"), "--out", out]
  r = subprocess.run(cmd, env=dict(os.environ, OMP_NUM_THREADS="2"), capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  for res in torch.load(out, weights_only=False):
    assert res["shape"][0] == 2
    assert res["fwd"] < 1e-5 and res["dx"] < 1e-4 and res["dw"] < 1e-4, res
    # AdamW over the rank-local expert region + the sharded router equals the single-rank update
    assert res["local_region"] > 0 and res["opt"] < 1e-5 and res["norm"] < 1e-4, res


def test_tensor_parallel_two_ranks_cpu(tmp_path):
  """Head- and hidden-sharded decoder equals the full model: logits, replicated and sharded gradients."""
  out = str(tmp_path / "tp.pt")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", "29661", os.path.join(HERE, "_tp_worker.py"), "--out", out]
  r = subprocess.run(cmd, env=dict(os.environ, OMP_NUM_THREADS="2"), capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  for res in torch.load(out, weights_only=False):
    assert res["fwd"] < 1e-4 and res["d_embed"] < 1e-5 and res["d_norm"] < 1e-5 and res["d_down"] < 1e-5, res
    # vocabulary-parallel lm_head: logits, log-probs, entropy and their gradients equal the unsharded head
    assert res["vp_logits"] < 1e-4 and res["vp_logp"] < 1e-4 and res["vp_ent"] < 1e-4, res
    assert res["vp_dhead"] < 1e-4 and res["vp_dembed"] < 1e-4, res


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
def test_sequence_parallel_two_ranks_cpu(tmp_path, layout):
  """Rows split along the sequence over 2 ranks (all-gathered K/V, causal prefix) give the full model's logits
  and, after the gradient reduction over the axis, its parameter gradients."""
  out = str(tmp_path / "sp.pt")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", "29671", os.path.join(HERE, "_sp_worker.py"), "--out", out,
         "--layout", layout]
  r = subprocess.run(cmd, env=dict(os.environ, OMP_NUM_THREADS="2"), capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  for res in torch.load(out, weights_only=False):
    assert res["fwd"] < 1e-4 and res["grads"] < 1e-4, res
