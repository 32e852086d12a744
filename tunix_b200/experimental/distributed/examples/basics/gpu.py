"""A body that joins the process group and reports its GPU: the counterpart of the reference's accelerator example
(tunix/experimental/distributed/examples/basics/tpu.py), with CUDA_VISIBLE_DEVICES in the role of the TPU
visibility variables.

  One process per GPU of this machine, rendezvous on the loopback address:

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29511 \\
        -m tunix_b200.experimental.distributed.runtime.main \\
        --process_main=tunix_b200.experimental.distributed.examples.basics.gpu.main

  Two jobs that split one machine:

    CUDA_VISIBLE_DEVICES=0,1 python -m torch.distributed.run --nproc-per-node 2 ... (as above, another port)
    CUDA_VISIBLE_DEVICES=2,3 python -m torch.distributed.run --nproc-per-node 2 ...

Without a GPU it joins a gloo group and says so.
"""
import argparse


def describe(ctx) -> str:
  import torch
  import torch.distributed as dist
  ctx.dist.initialize()
  where = f"rank {ctx.dist.rank} of {ctx.dist.world_size} ({dist.get_backend()})"
  if not torch.cuda.is_available():
    return f"{where}: no GPU visible, running on CPU"
  index = torch.cuda.current_device()
  props = torch.cuda.get_device_properties(index)
  probe = torch.ones(1, device="cuda") * (ctx.dist.rank + 1)
  dist.all_reduce(probe)                                    # proves that the group spans the GPUs
  return (f"{where}: cuda:{index} {props.name}, {props.total_memory / 2**30:.0f} GiB, sm_{props.major}{props.minor}, "
          f"{props.multi_processor_count} SMs; all-reduce of rank+1 = {probe.item():.0f}")


def main(ctx, argv) -> str:
  argparse.ArgumentParser().parse_args(argv)
  line = describe(ctx)
  print(line)
  return line
