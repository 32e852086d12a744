"""Two gloo ranks on CPU run GRPO through RLCluster with a sharded actor and a shared-storage rollout."""
import os
import subprocess
import sys

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
