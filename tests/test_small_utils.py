"""Small utility modules: env probes, compat helpers, sharding by spec, chunked application, wire-safety check,
experimental metric containers."""
import dataclasses

import numpy as np
import pytest
import torch

from tunix_b200.experimental.common import batch_utils, rpc_utils
from tunix_b200.experimental.metrics import metrics as xmetrics
from tunix_b200.utils import compat, env_utils, sharding_utils


def test_env_probes_are_consistent(monkeypatch):
  monkeypatch.delenv("RANK", raising=False)
  assert not env_utils.launched_by_torchrun()
  monkeypatch.setenv("RANK", "3"); monkeypatch.setenv("WORLD_SIZE", "8"); monkeypatch.setenv("LOCAL_RANK", "3")
  assert env_utils.launched_by_torchrun() and env_utils.rank_info() == {"rank": 3, "world_size": 8, "local_rank": 3}
  assert env_utils.is_pathways_initialized() is False and env_utils.is_internal_env() is False
  env_utils.setup_sharding_environment()
  import os
  assert os.environ["MASTER_ADDR"]
  assert isinstance(env_utils.peer_access_matrix(), list)


def test_alias_init_param_and_set_mesh():
  class A:
    @compat.alias_init_param("old", "new")
    def __init__(self, new=1):
      self.new = new
  assert A(old=5).new == 5 and A(new=6).new == 6 and A().new == 1
  with pytest.raises(ValueError, match="not both"):
    A(old=1, new=2)
  from tunix_b200.dist import mesh as mesh_lib
  m = mesh_lib.Mesh((1,), ("fsdp",), build_groups=False)
  with compat.set_mesh(m):
    assert mesh_lib.current_mesh() is m
  assert mesh_lib.current_mesh() is not m


def test_shard_without_mesh_is_identity():
  x = torch.arange(12).reshape(3, 4)
  assert sharding_utils.shard(x, ("fsdp", None)) is x


def test_apply_chunked_equals_one_call():
  a, b = np.arange(10.0).reshape(10, 1), np.arange(10.0, 20.0).reshape(10, 1)
  calls = []
  def fn(x, y):
    calls.append(len(x))
    return x * 2 + y
  want = fn(a, b)
  calls.clear()
  got = batch_utils.apply_chunked(fn, 4, a, b)
  assert calls == [4, 4, 2] and np.array_equal(got, want)
  assert np.array_equal(batch_utils.apply_chunked(fn, None, a, b), want)
  with pytest.raises(ValueError, match="disagree"):
    batch_utils.apply_chunked(fn, 2, a, b[:5])
  with pytest.raises(ValueError, match="positive"):
    batch_utils.apply_chunked(fn, 0, a, b)
  with pytest.raises(ValueError, match="batch dimension"):
    batch_utils.apply_chunked(fn, 2, np.float32(1.0))


def test_wire_safety_walks_nested_payloads():
  @dataclasses.dataclass
  class Msg:
    a: object
    b: object
  ok = Msg({"k": [np.zeros(3), (1, "x")]}, None)
  ok.b = ok          # a cycle
  rpc_utils.validate_wire_safe(ok)
  with pytest.raises(TypeError, match="torch.Tensor"):
    rpc_utils.validate_wire_safe(Msg({"k": [torch.zeros(2)]}, 1))
  sent = rpc_utils.to_wire(Msg({"k": [torch.ones(2, dtype=torch.bfloat16)]}, (torch.zeros(1),)))
  rpc_utils.validate_wire_safe(sent)
  assert sent.a["k"][0].dtype == np.float32 and isinstance(sent.b, tuple)


def test_weighted_metric_and_buffer():
  m = xmetrics.WeightedMetric(torch.tensor(6.0), torch.tensor(3.0))
  assert float(m.compute()) == 2.0
  assert float(xmetrics.WeightedMetric(1.0, 0.0).compute()) == 0.0
  assert float(xmetrics.WeightedMetric(1.0, 0.0, min_denom=2.0).compute()) == 0.5
  b1 = xmetrics.MetricsBuffer(1, {"loss": m}, {"kl": torch.tensor(1.0)}, {"kl": np.mean})
  b2 = xmetrics.MetricsBuffer(1, {"loss": xmetrics.WeightedMetric(2.0, 1.0)}, {"kl": 3.0})
  host = b1.merge(b2).to_host()
  assert host == {"loss": 2.0, "kl": 2.0}
