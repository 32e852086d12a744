"""Throughput of the host-staged weight transport (`experimental/orchestrator/host_staged_handler.py`) on one
machine: device -> pinned host -> TCP loopback -> pinned host -> device, one source endpoint and N destination
endpoints pulling in parallel. Prints one JSON line.

    python benchmarks/host_staged_transport_bench.py --gb 4 --destinations 2
"""
import argparse
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gb", type=float, default=2.0, help="bytes of weights per destination")
  ap.add_argument("--tensor-mb", type=int, default=256)
  ap.add_argument("--destinations", type=int, default=1)
  ap.add_argument("--rounds", type=int, default=3)
  ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
  a = ap.parse_args()
  from tunix_b200.experimental.orchestrator import host_staged_handler as hs, peer_memory_handler as pmh, weight_sync as ws
  dev = torch.device(a.device)
  per = a.tensor_mb * 2**20 // 2
  count = max(1, int(a.gb * 2**30 // (per * 2)))
  source = {f"w{i}": torch.randn(per, device=dev, dtype=torch.float32).to(torch.bfloat16) for i in range(count)}
  src = ws.WorkUnitId("trainer", "t", 0)
  endpoints = [hs.HostStagedEndpoint()]
  endpoints[0].attach(src, source)
  handler = hs.HostStagedHandler({src: endpoints[0].address}, timeout_s=600)
  handler.register_work_unit(pmh.manifest_of(src, source))
  dsts, stagings = [], []
  for d in range(a.destinations):
    unit = ws.WorkUnitId("rollout", f"r{d}", d)
    staging = {n: torch.zeros_like(t) for n, t in source.items()}
    ep = hs.HostStagedEndpoint()
    ep.attach(unit, staging)
    endpoints.append(ep)
    handler.register_endpoint(unit, ep.address)
    handler.register_work_unit(pmh.manifest_of(unit, staging))
    dsts.append(unit)
    stagings.append(staging)
  times = []
  for r in range(a.rounds + 1):                     # the first round allocates the pinned buffers: not timed
    t0 = time.perf_counter()
    result = handler.transfer([src], dsts, f"round-{r}")
    if dev.type == "cuda":
      torch.cuda.synchronize()
    assert result.success, result.message
    if r:
      times.append(time.perf_counter() - t0)
  ok = all(torch.equal(stagings[-1][n], source[n]) for n in source)
  nbytes = count * per * 2
  best = min(times)
  print(json.dumps({"metric": "host-staged weight transport, bytes delivered per second (all destinations)",
                    "value": a.destinations * nbytes / best / 1e9, "unit": "GB/s", "per_destination_gb": nbytes / 1e9,
                    "destinations": a.destinations, "tensor_mb": a.tensor_mb, "seconds_best": best,
                    "seconds_all": times, "device": str(dev), "bytes_equal": ok}))
  for ep in endpoints:
    ep.close()


if __name__ == "__main__":
  main()
