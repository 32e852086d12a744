"""Times the peer-memory collectives of the sharded optimizer step against NCCL.

  torchrun --nproc-per-node N --master-addr 127.0.0.1 -m benchmarks.p2p_bench [--params 2e9]

For a flat model of `--params` parameters it times, per optimizer step and per rank: the fused
reduce-scatter (pull the own shard of every peer's fp32 gradient and sum it, with the partial sums
of squares for the global norm), the fused AdamW + all-gather (update the own shard and store the
new bf16 values into every rank's replica), the GEMM with an all-reduce epilogue for a decode-sized
row-parallel projection, the GEMM that all-gathers its row-sharded weight inside the kernel, and the NCCL
collectives that move the same bytes. CUDA events around
`--iters` repetitions after warm-up, max over ranks. Bandwidth = bytes that cross NVLink per rank
and direction divided by the time; the roofline is the measured peer-copy bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters, warmup=3):
  for _ in range(warmup):
    fn()
  torch.cuda.synchronize()
  dist.barrier()
  a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  a.record()
  for _ in range(iters):
    fn()
  b.record()
  torch.cuda.synchronize()
  t = torch.tensor([a.elapsed_time(b) / iters], device="cuda")
  dist.all_reduce(t, op=dist.ReduceOp.MAX)
  return float(t)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--params", type=float, default=2e9)
  ap.add_argument("--iters", type=int, default=5)
  ap.add_argument("--link-gbs", type=float, default=770.0, help="measured peer-copy bandwidth per direction")
  ap.add_argument("--gemm-tflops", type=float, default=1674.5, help="measured cuBLAS bf16 burst rate")
  a = ap.parse_args()
  from tunix_b200 import optim
  from tunix_b200.dist import mesh as mesh_lib, symm as symm_lib
  from tunix_b200.ops import _lib
  local = int(os.environ.get("LOCAL_RANK", "0"))
  torch.cuda.set_device(local)
  dev = torch.device("cuda", local)
  mesh_lib.init_distributed("nccl")
  world, rank = dist.get_world_size(), dist.get_rank()
  n = int(a.params) // (1024 * world) * (1024 * world)
  shard = n // world
  sb = symm_lib.SymmetricBuffers(dist.group.WORLD, dev)
  grad = sb.alloc("grad", n, torch.float32)
  param = sb.alloc("param", n, torch.bfloat16)
  sb.rendezvous()
  grad.normal_()
  param.zero_()
  out = torch.empty(shard, dtype=torch.float32, device=dev)
  rows = []

  ms = _time(lambda: sb.reduce_scatter_sum(grad, out, rank), a.iters)
  link = (world - 1) * shard * 4                      # bytes this rank reads from peers
  rows.append({"op": "reduce_scatter_sum_f32 (peer pull + sum)", "ms": ms, "nvlink_GB_s": link / ms / 1e6,
               "frac_of_link": link / ms / 1e6 / a.link_gbs})
  nccl_out = torch.empty(shard, dtype=torch.float32, device=dev)
  ms = _time(lambda: dist.reduce_scatter_tensor(nccl_out, grad), a.iters)
  rows.append({"op": "nccl reduce_scatter fp32", "ms": ms, "nvlink_GB_s": link / ms / 1e6})

  tx = optim.adamw(1e-4, weight_decay=0.1)
  inner = getattr(tx, "inner", tx)
  state = {"master": {"flat": torch.zeros(shard, device=dev)}, "mu": {"flat": torch.zeros(shard, device=dev)},
           "nu": {"flat": torch.zeros(shard, device=dev)}, "count": torch.tensor(0, dtype=torch.int32)}
  scale = torch.ones(1, device=dev)
  sl = slice(rank * shard, (rank + 1) * shard)
  ms = _time(lambda: sb.adamw_allgather(inner, state, out, param, sl, scale), a.iters)
  link = (world - 1) * shard * 2                      # bf16 values this rank stores into peers
  rows.append({"op": "adamw_allgather (update shard + peer push)", "ms": ms, "nvlink_GB_s": link / ms / 1e6,
               "frac_of_link": link / ms / 1e6 / a.link_gbs,
               "note": "also streams 28 B/param of local optimizer state"})
  ms = _time(lambda: dist.all_gather_into_tensor(param, param[sl].clone()), a.iters)
  rows.append({"op": "nccl all_gather bf16", "ms": ms, "nvlink_GB_s": link / ms / 1e6})

  # decode-sized row-parallel projection: [64, K/world] x [4096, K/world]^T summed over ranks
  M, N, K = 64, 4096, 12288 // world
  x = torch.randn(M, K, device=dev).bfloat16()
  w = torch.randn(N, K, device=dev).bfloat16()
  ws = sb.alloc("sum", M * N, torch.float32)
  sb.rendezvous()
  lib = _lib.require()
  y = torch.empty(M, N, dtype=torch.bfloat16, device=dev)

  def fused():
    ws.zero_()
    sb.barrier()
    rc = lib.tx_gemm_bf16_allreduce(x.data_ptr(), w.data_ptr(), symm_lib._ptr_array(sb.peer_ptrs["sum"]), world, M,
                                    N, K, K, K, 0, 0, 1.0, _lib.status_word(dev).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "tx_gemm_bf16_allreduce")
    sb.barrier()
    _lib.check_rc(lib.tx_f32_sum_to_bf16(ws.data_ptr(), y.data_ptr(), N, M, N, _lib.stream_ptr()), "finish")

  def plain():
    t = torch.nn.functional.linear(x, w)
    dist.all_reduce(t)
    return t
  ms_f = _time(fused, 20)
  ms_p = _time(plain, 20)
  ref = plain().float()
  fused()
  torch.cuda.synchronize()
  err = float((y.float() - ref).abs().max() / ref.abs().max())
  rows.append({"op": f"gemm + all-reduce epilogue M={M} N={N} K={K}/rank", "ms": ms_f, "rel_err_vs_nccl": err})
  rows.append({"op": "library linear + nccl all_reduce (same shape)", "ms": ms_p})
  # all-gather fused into the consuming GEMM: Llama-3.1-8B gate|up half (N 14336, K 4096) on 8192 tokens, the
  # weight row-sharded over the ranks. Roofline: the slower of the GEMM at the measured cuBLAS rate and the
  # remote shards over the link.
  from tunix_b200.ops import kernels
  Mg, Ng, Kg = 8192, 14336, 4096
  if Ng % (128 * world) == 0:
    per = Ng // world
    wsh = sb.alloc("wshard", per * Kg, torch.bfloat16).view(per, Kg)
    sb.rendezvous()
    wsh.copy_((torch.randn(per, Kg, device=dev) * 0.02).bfloat16())
    xa = torch.randn(Mg, Kg, device=dev).bfloat16()
    stage = torch.empty(Ng, Kg, dtype=torch.bfloat16, device=dev)
    cnt = torch.empty(Ng // 128, dtype=torch.int32, device=dev)
    cg = torch.empty(Mg, Ng, dtype=torch.bfloat16, device=dev)
    wfull = torch.empty(Ng, Kg, dtype=torch.bfloat16, device=dev)
    ptrs = sb.peer_ptrs["wshard"]
    sb.barrier()

    def fused_ag():
      kernels.gemm_allgather_b(xa, ptrs, rank, per, stage, cnt, out=cg)

    def plain_ag():
      dist.all_gather_into_tensor(wfull, wsh)
      kernels.gemm(xa, wfull, out=cg)

    def gemm_only():
      kernels.gemm(xa, wfull, out=cg)
    ms_f = _time(fused_ag, 10)
    got = cg.float().clone()
    ms_p = _time(plain_ag, 10)
    err = float((got - cg.float()).abs().max() / cg.float().abs().max())
    ms_g = _time(gemm_only, 10)
    fl = 2.0 * Mg * Ng * Kg
    link = (world - 1) * per * Kg * 2
    t_roof = max(fl / (a.gemm_tflops * 1e12), link / (a.link_gbs * 1e9)) * 1e3
    rows.append({"op": f"all-gather fused into GEMM M={Mg} N={Ng} K={Kg}", "ms": ms_f, "tflops": fl / ms_f / 1e9,
                 "nvlink_GB_s": link / ms_f / 1e6, "roofline_ms": t_roof, "frac_of_roofline": t_roof / ms_f,
                 "rel_err_vs_nccl_path": err})
    rows.append({"op": "nccl all_gather + tcgen05 GEMM (same shape)", "ms": ms_p, "tflops": fl / ms_p / 1e9})
    rows.append({"op": "tcgen05 GEMM alone on the gathered weight", "ms": ms_g, "tflops": fl / ms_g / 1e9})
  _lib.check_status()
  if rank == 0:
    for r in rows:
      print(json.dumps({"world": world, "params": n, **{k: (round(v, 4) if isinstance(v, float) else v)
                                                        for k, v in r.items()}}), flush=True)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
