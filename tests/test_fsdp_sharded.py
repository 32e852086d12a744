"""Sharded-parameter FSDP (`dist/fsdp_sharded.py`): equality with the resident store on gloo ranks, whole-model
access, checkpoints, and the stated limits. The 2-GPU version is in tests/test_gpu_fsdp.py."""
import os
import subprocess
import sys

import pytest
import torch

from tunix_b200 import optim
from tunix_b200.common.configs import TrainingConfig
from tunix_b200.dist import fsdp, fsdp_sharded
from tunix_b200.models.transformer import ModelConfig, RematConfig, Transformer
from tunix_b200.sft.peft_trainer import PeftTrainer, TrainingInput

HERE = os.path.dirname(os.path.abspath(__file__))


def _worker(tmp_path, tag, nproc, port, *extra):
  out = str(tmp_path / f"{tag}.pt")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr",
         "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "_fsdp_worker.py"), "--out", out, "--device", "cpu",
         "--layers", "3", *extra]
  r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
  assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
  return torch.load(out, weights_only=False)


def test_sharded_parameters_train_like_the_resident_store_on_two_ranks(tmp_path):
  resident = _worker(tmp_path, "resident", 2, 29741, "--mode", "resident")
  sharded = _worker(tmp_path, "sharded", 2, 29742, "--mode", "sharded", "--remat", "1")
  for n, p in resident["params"].items():
    rel = (p - sharded["params"][n]).norm() / (p.norm() + 1e-9)
    assert rel < 1e-5, (n, float(rel))
  assert resident["loss"] == pytest.approx(sharded["loss"], rel=1e-5)
  mem = sharded["memory"]
  assert mem["param_shard"] == pytest.approx(mem["grad_shard"])          # fp32 model on CPU: same bytes
  # half of the layers' parameters per rank, while the two slots hold one layer each
  assert mem["slots"] < 2.5 * mem["param_shard"]


def _tiny(remat=RematConfig.NONE, layers=3):
  cfg = ModelConfig(num_layers=layers, vocab_size=64, embed_dim=32, hidden_dim=48, num_heads=4, head_dim=8,
                    num_kv_heads=2, remat_config=remat, max_position=32)
  return Transformer(cfg).init_weights(seed=0, scale=0.2)


def _batches(n, seed=3):
  g = torch.Generator().manual_seed(seed)
  return [TrainingInput(torch.randint(0, 64, (2, 16), generator=g), torch.ones(2, 16)) for _ in range(n)]


def test_whole_model_access_and_writeback():
  model = _tiny()
  before = {n: p.detach().clone() for n, p in model.named_parameters()}
  fsdp.shard_model(model, None, mode="sharded")
  store = model.flat_store
  assert isinstance(store, fsdp_sharded.ShardedParamStore) and not store.resident
  assert len(store.units) == 3 and all(p.grad_managed for u in store.units for p, _, _ in u.params)
  with pytest.raises(AttributeError, match="summon_full_params"):
    store.flat_param
  with store.summon_full_params():
    for n, p in model.named_parameters():
      assert torch.equal(p.detach(), before[n]), n
  # a forward pass gathers what it needs by itself and gives the same logits as an untouched copy
  tokens = torch.randint(0, 64, (2, 12), generator=torch.Generator().manual_seed(1))
  with torch.no_grad():
    got = model(tokens)[0]
    want = _tiny()(tokens)[0]
  assert torch.allclose(got, want, atol=1e-6)
  with store.summon_full_params(writeback=True):
    with torch.no_grad():
      model.layers[1].attn.o_proj.w.mul_(2.0)
  with store.summon_full_params():
    assert torch.equal(model.layers[1].attn.o_proj.w.detach(), 2.0 * before["layers.1.attn.o_proj.w"])
    assert torch.equal(model.layers[2].attn.o_proj.w.detach(), before["layers.2.attn.o_proj.w"])


def test_checkpoint_round_trip_and_optimizer_state_in_sharded_mode(tmp_path):
  tc = TrainingConfig(eval_every_n_steps=100, gradient_accumulation_steps=2, max_grad_norm=1.0, pbar_description=None,
                      checkpoint_root_directory=str(tmp_path / "ckpt"))
  model = fsdp.shard_model(_tiny(), None, mode="sharded")
  tr = PeftTrainer(model, optim.adamw(5e-3, weight_decay=0.01), tc)
  tr.train(_batches(4))
  tr.close() if hasattr(tr, "close") else None
  with model.flat_store.summon_full_params():
    trained = {n: p.detach().clone() for n, p in model.named_parameters()}
  fresh = fsdp.shard_model(_tiny(), None, mode="sharded")
  tr2 = PeftTrainer(fresh, optim.adamw(5e-3, weight_decay=0.01), tc)
  assert tr2.train_steps == 2
  with fresh.flat_store.summon_full_params():
    for n, p in fresh.named_parameters():
      assert torch.allclose(p.detach(), trained[n], atol=1e-6), n
  # and the same run without any store ends on the same weights
  plain = _tiny()
  tc2 = TrainingConfig(eval_every_n_steps=100, gradient_accumulation_steps=2, max_grad_norm=1.0, pbar_description=None)
  PeftTrainer(plain, optim.adamw(5e-3, weight_decay=0.01), tc2).train(_batches(4))
  for n, p in plain.named_parameters():
    assert torch.allclose(p.detach(), trained[n], atol=2e-5), n


def test_whole_decoder_recomputation_is_refused():
  model = fsdp.shard_model(_tiny(remat=RematConfig.DECODER), None, mode="sharded")
  tokens = torch.randint(0, 64, (2, 12), generator=torch.Generator().manual_seed(1))
  logits = model(tokens)[0]
  with pytest.raises(RuntimeError, match="per-block recomputation only"):
    logits.float().sum().backward()
