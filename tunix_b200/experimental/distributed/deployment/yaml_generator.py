"""Renders a Kubernetes JobSet manifest for a B200 (or CPU) worker group.

  python -m tunix_b200.experimental.distributed.deployment.yaml_generator \
      yamls/jobset.gpu.yaml --gpu_slice b200:2x8 --worker_container_image IMG \
      --worker_startup_command "python -m tunix_b200.cli.grpo_main cfg.yaml"

``--gpu_slice TYPE:NODESxGPUS`` names the accelerator, the number of nodes and
GPUs per node; one pod runs per node with every GPU of the node, and the
startup command is wrapped in ``torch.distributed.run`` with a static
rendezvous on pod 0 so NCCL sees one rank per GPU. Templates use
``string.Template`` placeholders.

Counterpart of tunix/experimental/distributed/deployment/yaml_generator.py
(TPU slices and Pathways sidecars there; NVLink domains here).
"""

from __future__ import annotations

import argparse
import os
import string
import sys

GPU_TYPES = {
    # type -> (node selector value, GPUs per node, instance type)
    "b200": ("nvidia-b200", 8, "a4-highgpu-8g"),
    "gb200": ("nvidia-gb200", 4, "a4x-highgpu-4g"),
    "h200": ("nvidia-h200-141gb", 8, "a3-ultragpu-8g"),
    "h100": ("nvidia-h100-80gb", 8, "a3-highgpu-8g"),
}


def parse_gpu_slice(spec: str | None):
  """'b200:2x8' -> dict(type, accelerator, machine, nodes, gpus_per_node)."""
  if not spec or spec == ":":
    return None
  gpu_type, _, shape = spec.partition(":")
  if gpu_type not in GPU_TYPES:
    raise ValueError(
        f"Unsupported GPU type {gpu_type!r}; known: {sorted(GPU_TYPES)}")
  accel, per_node, machine = GPU_TYPES[gpu_type]
  if not shape:
    nodes, gpus = 1, per_node
  else:
    dims = shape.lower().split("x")
    if len(dims) != 2 or not all(d.isdigit() and int(d) > 0 for d in dims):
      raise ValueError(f"GPU slice shape '{shape}' is not NODESxGPUS")
    nodes, gpus = int(dims[0]), int(dims[1])
  if gpus > per_node:
    raise ValueError(f"{gpu_type} nodes have {per_node} GPUs, asked for {gpus}")
  if nodes > 1 and gpus != per_node:
    raise ValueError("multi-node slices must use every GPU of each node")
  return dict(type=gpu_type, accelerator=accel, machine=machine, nodes=nodes,
              gpus_per_node=gpus)


def render(template_text: str, args: argparse.Namespace, environ=None) -> str:
  env = os.environ if environ is None else environ
  sl = parse_gpu_slice(args.gpu_slice)
  user = env.get("USER", "user")
  name = args.jobset_name
  if name is None:
    name = (f"{user}-{sl['type']}-{sl['nodes'] * sl['gpus_per_node']}"
            if sl else f"{user}-cpu")
  nodes = sl["nodes"] if sl else 1
  gpus = sl["gpus_per_node"] if sl else 0
  launch = args.worker_startup_command
  if sl and args.wrap_torchrun:
    launch = (
        "python -m torch.distributed.run"
        f" --nnodes={nodes} --nproc-per-node={gpus}"
        " --node-rank=$JOB_COMPLETION_INDEX"
        f" --master-addr={name}-proc-0-0.{name}"
        f" --master-port={args.rendezvous_port} " + launch)
  values = dict(
      JOBSET_NAME=name, USER=user, CPU_MACHINE=args.cpu_machine,
      GPU_MACHINE=sl["machine"] if sl else None,
      GPU_ACCELERATOR=sl["accelerator"] if sl else None,
      GPU_TYPE=sl["type"] if sl else None,
      GPUS_PER_NODE=gpus, NUM_NODES=nodes, REPLICAS=1, COMPLETIONS=nodes,
      PARALLELISM=nodes, USER_CONTAINER=args.worker_container_name,
      USER_CONTAINER_IMAGE=args.worker_container_image,
      USER_CONTAINER_PORT=args.worker_container_port,
      RENDEZVOUS_PORT=args.rendezvous_port,
      SHM_SIZE=args.shm_size,
      STARTUP_COMMAND=launch.replace("\n", " "))
  return string.Template(template_text).substitute(values)


def build_parser() -> argparse.ArgumentParser:
  p = argparse.ArgumentParser(
      description="Generate a Kubernetes JobSet YAML from a template.")
  p.add_argument("template_file")
  p.add_argument("--jobset_name", default=None)
  p.add_argument("--gpu_slice", default=None,
                 help="TYPE:NODESxGPUS, e.g. b200:2x8; types: "
                 + ", ".join(sorted(GPU_TYPES)))
  p.add_argument("--cpu_machine", default=None, help="e.g. n2-standard-64")
  p.add_argument("--worker_container_name", default="main")
  p.add_argument("--worker_container_image", default="python:3.12")
  p.add_argument("--worker_container_port", type=int, default=12345)
  p.add_argument("--rendezvous_port", type=int, default=29500)
  p.add_argument("--shm_size", default="64Gi")
  p.add_argument("--worker_startup_command", default="sleep infinity")
  p.add_argument("--no_torchrun", dest="wrap_torchrun", action="store_false",
                 help="run the startup command as is, one process per pod")
  p.add_argument("-o", "--output", default=None)
  return p


def main(argv=None) -> None:
  args = build_parser().parse_args(argv)
  with open(args.template_file, "r", encoding="utf-8") as f:
    text = render(f.read(), args)
  if args.output:
    with open(args.output, "w", encoding="utf-8") as f:
      f.write(text)
  else:
    sys.stdout.write(text)


if __name__ == "__main__":
  main()
