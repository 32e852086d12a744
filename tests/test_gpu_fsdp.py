"""Sharded-vs-unsharded equivalence of FSDP training on 2 GPUs, for both transports
(NCCL collectives and the peer-memory kernels)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, out, transport, port, args=(), **extra_env):
  env = dict(os.environ, NCCL_NVLS_ENABLE="0", TUNIX_PEER_WAIT_MS="20000", **extra_env)
  if nproc == 1:
    cmd = [sys.executable, os.path.join(HERE, "_fsdp_worker.py"), "--out", out, "--transport", transport, *args]
  else:
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_fsdp_worker.py"),
           "--out", out, "--transport", transport, *args]
  r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  return torch.load(out, weights_only=False)


@pytest.mark.parametrize("transport", ["nccl", "p2p"])
def test_fsdp2_matches_single_gpu(kernel_lib, tmp_path, transport):
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  ref = _run(1, str(tmp_path / "ref.pt"), "local", 0)
  got = _run(2, str(tmp_path / f"{transport}.pt"), transport, 29611 if transport == "nccl" else 29612)
  for n, p in ref["params"].items():
    q = got["params"][n]
    rel = (p - q).norm() / (p.norm() + 1e-6)
    assert rel < 2e-2, (n, rel.item())
  assert abs(ref["loss"][-1] - got["loss"][-1]) < 0.05


def test_sharded_parameters_match_the_resident_store_on_gpus(kernel_lib, tmp_path):
  """Parameters, gradients and optimizer state all sharded (`dist/fsdp_sharded.py`): layers gathered on a side
  stream for forward and backward, gradients reduce-scattered per layer. One GPU must reproduce the resident
  store (same kernels, same order); two GPUs must agree with it like the resident 2-GPU run does."""
  args = ("--layers", "4")
  ref = _run(1, str(tmp_path / "ref.pt"), "local", 0, args)
  one = _run(1, str(tmp_path / "one.pt"), "local", 0, args + ("--mode", "sharded"))
  for n, p in ref["params"].items():      # same kernels; only the grouping of the norm's partial sums may differ
    rel = (p - one["params"][n]).norm() / (p.norm() + 1e-6)
    assert rel < 2e-3, (n, rel.item())
  if torch.cuda.device_count() < 2:
    return
  two = _run(2, str(tmp_path / "two.pt"), "nccl", 29616, args + ("--mode", "sharded"))
  for n, p in ref["params"].items():
    rel = (p - two["params"][n]).norm() / (p.norm() + 1e-6)
    assert rel < 2e-2, (n, rel.item())
  assert abs(ref["loss"][-1] - two["loss"][-1]) < 0.05
  assert two["memory"]["param_shard"] < 0.6 * one["memory"]["param_shard"]


def test_fsdp2_on_the_own_peer_allocator(kernel_lib, tmp_path):
  """The same equivalence with the symmetric buffers coming from `dist/vmm.py` (cuMemCreate, descriptors over Unix
  sockets, cuMemMap) instead of torch's symmetric-memory plumbing."""
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  ref = _run(1, str(tmp_path / "ref.pt"), "local", 0)
  got = _run(2, str(tmp_path / "vmm.pt"), "p2p", 29613, TUNIX_B200_SYMM_BACKEND="vmm")
  for n, p in ref["params"].items():
    rel = (p - got["params"][n]).norm() / (p.norm() + 1e-6)
    assert rel < 2e-2, (n, rel.item())
  assert abs(ref["loss"][-1] - got["loss"][-1]) < 0.05


def test_grpo_data_parallel_two_gpus(kernel_lib, tmp_path):
  """GRPO through RLCluster on 2 GPUs: sharded actor state, rollout on the trainer's replica."""
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  out = str(tmp_path / "grpo.pt")
  env = dict(os.environ, NCCL_NVLS_ENABLE="0", TUNIX_PEER_WAIT_MS="20000")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", "29613", os.path.join(HERE, "_grpo_dp_worker.py"), "--out", out,
         "--device", "cuda"]
  r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  got = torch.load(out, weights_only=False)
  assert got["steps"] == 2 and got["moved"] > 0
  assert abs(got["checksums"][0] - got["checksums"][1]) < 1e-6 * max(1.0, abs(got["checksums"][0]))


def test_tensor_parallel_fused_allreduce_two_gpus(kernel_lib, tmp_path):
  """TP=2 decoder whose row-parallel exits add their GEMM tiles into both ranks' buffers over NVLink."""
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  out = str(tmp_path / "tp.pt")
  env = dict(os.environ, NCCL_NVLS_ENABLE="0", TUNIX_PEER_WAIT_MS="20000")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", "29614", os.path.join(HERE, "_tp_worker.py"), "--out", out, "--device", "cuda"]
  r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  for res in torch.load(out, weights_only=False):
    assert res["grad_ok"]
    assert max(res["fwd0"], res["fwd1"], res["fwd2"]) < 3e-2, res
    assert res["vp_logp"] < 2e-2 and res["vp_ent"] < 2e-2 and res["vp_dh"] < 3e-2 and res["vp_dw"] < 3e-2, res


def test_moe_expert_parallel_peer_memory_two_gpus(kernel_lib, tmp_path):
  """Expert parallelism with our dispatch / combine kernels over NVLink peer memory and the grouped tcgen05 GEMM:
  outputs, input gradients, router and expert-weight gradients equal the unsharded layer on every rank."""
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  out = str(tmp_path / "ep.pt")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", "29615", os.path.join(HERE, "_moe_ep_worker.py"), "--out", out, "--device", "cuda"]
  env = dict(os.environ, NCCL_NVLS_ENABLE="0", TUNIX_PEER_WAIT_MS="20000")
  r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  for res in torch.load(out, weights_only=False):
    assert res["peer"], "the peer-memory path was not taken"
    for rnd in (0, 1):
      assert res[f"fwd{rnd}"] < 3e-2 and res[f"dx{rnd}"] < 3e-2, res
      assert res[f"dw{rnd}"] < 3e-2 and res[f"dwd{rnd}"] < 3e-2 and res[f"drouter{rnd}"] < 5e-2, res


def test_tensor_parallel_rollout_with_kernel_weight_sync_two_gpus(kernel_lib, tmp_path):
  """TP=2 rollout on slices produced by the re-sharding copy kernel (own and peer replica as source): slices equal
  the sliced model, both ranks sample the same tokens, their log-probs agree with the unsharded model's forward
  within the rollout tolerance, eagerly and under CUDA graphs, with the exits all-reducing inside the skinny GEMM."""
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  out = str(tmp_path / "tpr.pt")
  env = dict(os.environ, NCCL_NVLS_ENABLE="0", TUNIX_PEER_WAIT_MS="20000")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", "29617", os.path.join(HERE, "_tp_rollout_worker.py"), "--out", out]
  r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  for res in torch.load(out, weights_only=False):
    assert res["slice_err_own"] == 0.0 and res["slice_err_peer"] == 0.0, res
    for key in ("own_eager", "own_graph", "peer_eager", "peer_graph"):
      assert res[f"same_tokens_{key}"], res                # reduced logits are bitwise equal on the ranks of a group
      assert res[f"lp_err_{key}"] < 0.08, res
    assert res["captured_own_graph"] and res["captured_peer_graph"], res
    assert res["same_tokens_96"] and res["lp_err_96"] < 0.08, res
    assert abs(res["update_ratio"] - 1.5) < 0.02, res


@pytest.mark.parametrize("layout", ["contiguous", "zigzag"])
def test_sequence_parallel_peer_pull_two_gpus(kernel_lib, tmp_path, layout):
  """Rows split along the sequence over 2 GPUs; keys / values (and their gradients) move with the peer copy
  kernel. Logits and reduced parameter gradients equal the unsharded bf16 model's within bf16 error."""
  if torch.cuda.device_count() < 2:
    pytest.skip("needs 2 GPUs")
  out = str(tmp_path / "sp.pt")
  env = dict(os.environ, NCCL_NVLS_ENABLE="0", TUNIX_PEER_WAIT_MS="20000")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
         "127.0.0.1", "--master-port", "29641", os.path.join(HERE, "_sp_worker.py"), "--out", out, "--layout", layout,
         "--backend", "nccl"]
  r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
  for res in torch.load(out, weights_only=False):
    assert res["fwd"] < 3e-2 and res["grads"] < 6e-2, res
