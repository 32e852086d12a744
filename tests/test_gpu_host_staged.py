"""The host-staged weight transport with device tensors on both sides: device -> pinned host -> TCP (loopback) ->
pinned host -> device, double-buffered on each side."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_device_tensors_cross_the_host_staged_transport():
  from tunix_b200.experimental.orchestrator import host_staged_handler as hs, peer_memory_handler as pmh, weight_sync as ws
  dev = torch.device("cuda", 0)
  g = torch.Generator(device="cpu").manual_seed(11)
  shapes = {"embed": (4096, 512), "l0.qkv": (1536, 512), "l0.norm": (512,), "l1.qkv": (1536, 512), "l1.down": (512, 2048),
            "odd": (1001, 3), "scalar": ()}
  source = {n: torch.randn(s, generator=g).to(torch.bfloat16).to(dev) for n, s in shapes.items()}
  same = {n: torch.zeros(s, dtype=torch.bfloat16, device=dev) for n, s in shapes.items()}
  wide = {n: torch.zeros(s, dtype=torch.float32, device=dev) for n, s in shapes.items()}
  src, d1, d2 = ws.WorkUnitId("trainer", "t", 0), ws.WorkUnitId("rollout", "a", 0), ws.WorkUnitId("rollout", "b", 1)
  with hs.HostStagedEndpoint() as a, hs.HostStagedEndpoint() as b:
    a.attach(src, source, generation=3)
    b.attach(d1, same)
    b.attach(d2, wide)
    handler = hs.HostStagedHandler({src: a.address, d1: b.address, d2: b.address}, timeout_s=60)
    for unit, tensors in ((src, source), (d1, same), (d2, wide)):
      handler.register_work_unit(pmh.manifest_of(unit, tensors))
    result = handler.transfer([src], [d1, d2], "round-1", generation=3)
    assert result.success, result.message
    torch.cuda.synchronize()
    for n in shapes:
      assert torch.equal(same[n], source[n]), n
      assert torch.equal(wide[n], source[n].float()), n
    assert a.served["fetch"] == 2 and b.served["pull"] == 2
    # a second round with new values reuses the endpoints
    for t in source.values():
      t.add_(1.0)
    a.attach(src, source, generation=4)
    assert not handler.transfer([src], [d1], "round-2", generation=3).success      # stale
    assert handler.transfer([src], [d1], "round-2", generation=4).success
    torch.cuda.synchronize()
    assert all(torch.equal(same[n], source[n]) for n in shapes)
