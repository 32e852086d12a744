"""Child process of the host-staged transport test: holds one unit behind a `HostStagedEndpoint`, prints the
endpoint's port, and serves until its stdin closes."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def tensors(seed: int, dtype):
  g = torch.Generator().manual_seed(seed)
  shapes = {"embed": (64, 16), "layers.0.w": (16, 48), "layers.0.norm": (16,), "layers.1.w": (16, 48), "scalar": ()}
  return {n: (torch.randn(s, generator=g) if seed else torch.zeros(s)).to(dtype) for n, s in shapes.items()}


def main():
  role, unit, generation = sys.argv[1], sys.argv[2], int(sys.argv[3])
  from tunix_b200.experimental.orchestrator import host_staged_handler as hs
  held = tensors(7, torch.bfloat16) if role == "source" else tensors(0, torch.bfloat16 if role == "same" else torch.float32)
  with hs.HostStagedEndpoint() as ep:
    ep.attach(unit, held, generation if role == "source" else None)
    print(ep.address[1], flush=True)
    sys.stdin.read()            # the parent closes the pipe when it is done


if __name__ == "__main__":
  main()
