"""Checkpoint manager: policy-driven, asynchronous saves and restore-on-construction.

API and semantics follow tunix/sft/checkpoint_manager.py:98-331: checkpointables `model_params`
(+ `optimizer_state`), LoRA-only save / partial restore, custom metadata, `maybe_restore`
returning `(step, custom_metadata)`. Files are written in the Orbax directory layout
(`tunix_b200.ckpt.orbax_layout`).

A save first snapshots the tensors to host memory on the calling thread (so training may
overwrite the GPU copies immediately), then a background thread writes the files into
`<root>/<step>.tmp-*` and renames the directory into place - a step directory exists only
when complete.

Multi-rank jobs. Whether to save is decided once, by rank 0 of the group that shares the state
(its policy clock, its pending write), and broadcast, so the ranks never disagree about entering
a save. Replicated leaves are written by rank 0. Leaves that are sharded over the ranks
(`orbax_layout.ShardedArray`: the flat optimizer-state shards of `dist.fsdp`, expert-parallel
expert weights) are written by their owners as chunk files of one array - no state is gathered.
Each rank drops a marker into the temporary directory when its files are complete; rank 0
renames the directory once all markers are there, without any collective on the writer threads.
"""
from __future__ import annotations

import concurrent.futures as cf
import logging
import os
import shutil
import threading
import time
from typing import Any, Dict, Mapping, Optional, Tuple

import torch

from ..ckpt import layout, orbax_layout
from . import checkpoint_options

log = logging.getLogger(__name__)


def _group_rank_world(group) -> Tuple[int, int]:
  import torch.distributed as dist
  if group is None or not dist.is_available() or not dist.is_initialized():
    return 0, 1
  return dist.get_rank(group), dist.get_world_size(group)


def _share_from_rank0(values: Tuple[int, int], group, device) -> Tuple[int, int]:
  """Rank 0's (flag, timestamp) for every rank of `group`."""
  import torch.distributed as dist
  rank, world = _group_rank_world(group)
  if world == 1:
    return values
  dev = device if (device is not None and dist.get_backend(group) == "nccl") else "cpu"
  t = torch.tensor(list(values), dtype=torch.int64, device=dev)
  dist.broadcast(t, src=dist.get_global_rank(group, 0), group=group)
  a, b = t.tolist()
  return int(a), int(b)


def _snapshot(tree: Mapping[Any, Any], rank: int = 0) -> Dict[Any, Any]:
  """Device -> host copy of every leaf this rank has to write (pinned staging for CUDA tensors): all
  leaves on rank 0, only the sharded ones elsewhere."""
  from ..ckpt.orbax_layout import ShardedArray

  def to_host(t: torch.Tensor) -> torch.Tensor:
    t = torch.as_tensor(t).detach()
    if t.is_cuda:
      host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
      host.copy_(t, non_blocking=True)
      return host
    return t.clone()

  out = {}
  for k, t in tree.items():
    if isinstance(t, ShardedArray):
      out[k] = ShardedArray(to_host(t.local), t.global_shape, t.chunk_shape, t.chunk_index)
    elif rank == 0:
      out[k] = to_host(t)
  if torch.cuda.is_available():
    torch.cuda.current_stream().synchronize()
  return out


class CheckpointManager:
  """Saves and restores model parameters and optimizer state."""

  def __init__(self, root_directory: Optional[str] = None, options: Any = None):
    self._root = root_directory or None
    self._options = checkpoint_options.resolve_checkpointing_defaults(options)
    self._executor: Optional[cf.ThreadPoolExecutor] = None
    self._pending: Optional[cf.Future] = None
    self._last_save_time: Optional[float] = None
    self._last_saved_step: Optional[int] = None
    self._lock = threading.Lock()
    if self._root:
      os.makedirs(self._root, exist_ok=True)
      self._executor = cf.ThreadPoolExecutor(max_workers=1, thread_name_prefix="ckpt-writer")

  # ---- queries -------------------------------------------------------------------------
  def latest_step(self) -> Optional[int]:
    if not self._root:
      return None
    self.wait_until_finished()
    steps = orbax_layout.list_steps(self._root)
    return steps[-1] if steps else None

  def all_steps(self):
    return orbax_layout.list_steps(self._root) if self._root else []

  def wait_until_finished(self) -> None:
    p = self._pending
    if p is not None:
      timeout = self._options.async_options.timeout_secs if self._options.async_options else None
      p.result(timeout=timeout)
      self._pending = None

  # ---- save --------------------------------------------------------------------------------
  def _write(self, step: int, items: Dict[str, Dict[Any, Any]], extras: Dict[str, Dict[str, bytes]], custom_metadata,
             init_ns: int, rank: int = 0, world: int = 1) -> None:
    final = os.path.join(self._root, str(step))
    tmp = f"{final}.tmp-{init_ns}"
    try:
      for name, tree in items.items():
        orbax_layout.write_tree(os.path.join(tmp, name), tree, process_index=rank,
                                use_ocdbt=bool(getattr(self._options, "use_ocdbt", False)))
      with open(os.path.join(tmp, f"_rank_{rank}.done"), "w") as f:
        f.write("ok")
      if rank != 0:
        return
      # rank 0 commits once every rank's files are complete
      timeout = self._options.async_options.timeout_secs if self._options.async_options else None
      deadline = None if timeout is None else time.monotonic() + timeout
      missing = list(range(world))
      while missing:
        missing = [r for r in missing if not os.path.exists(os.path.join(tmp, f"_rank_{r}.done"))]
        if missing:
          if deadline is not None and time.monotonic() > deadline:
            raise TimeoutError(f"checkpoint {step}: ranks {missing} did not finish writing within {timeout} s")
          time.sleep(0.02)
      for r in range(world):
        os.remove(os.path.join(tmp, f"_rank_{r}.done"))
      for name, files in extras.items():
        for fname, data in files.items():
          with open(os.path.join(tmp, name, fname), "wb") as f:
            f.write(data)
      orbax_layout.write_checkpoint_metadata(tmp, list(items.keys()), custom_metadata, init_ns)
      if os.path.exists(final):
        shutil.rmtree(final)
      os.replace(tmp, final)
    finally:
      if rank == 0 and os.path.exists(tmp):
        shutil.rmtree(tmp, ignore_errors=True)
    policy = self._options.preservation_policy
    if policy is not None:
      for s in policy.to_delete(orbax_layout.list_steps(self._root)):
        shutil.rmtree(os.path.join(self._root, str(s)), ignore_errors=True)

  def _wants_to_save(self, step: int, force: bool) -> bool:
    if self._last_saved_step == step:
      return False
    if force:
      return True
    policy = self._options.save_decision_policy
    if (isinstance(policy, checkpoint_options.ContinuousCheckpointingPolicy) and self._pending is not None
        and not self._pending.done()):
      return False    # "as often as the writer allows": a save is still being written, so this step is skipped
    # every other policy names the steps it wants; `save` waits for the previous write instead of dropping one
    return bool(policy.should_save(step, self._last_saved_step, self._last_save_time))

  def save(self, step: int, model: torch.nn.Module, optimizer: Any = None, save_only_lora_params: bool = False,
           force: bool = False, custom_metadata: Optional[Mapping[str, Any]] = None) -> bool:
    """Saves the parameters (and optimizer state) for `step`. Returns whether a save was
    performed (synchronous mode) or started (asynchronous mode). In a multi-rank job every rank of the
    group that shares the state must call this for every step it is called on any rank: the decision is
    rank 0's and is broadcast."""
    if not self._root:
      return False
    group = getattr(optimizer, "checkpoint_group", lambda: None)() if optimizer is not None else None
    if group is None:
      store = getattr(model, "flat_store", None)
      group = store.group if store is not None and store.world > 1 else None
    rank, world = _group_rank_world(group)
    device = next((p.device for p in model.parameters() if p.is_cuda), None)
    go, init_ns = _share_from_rank0((int(self._wants_to_save(step, force)) if rank == 0 else 0, time.time_ns()),
                                    group, device)
    if not go:
      return False
    self.wait_until_finished()
    items: Dict[str, Dict[Any, Any]] = {}
    extras: Dict[str, Dict[str, bytes]] = {}
    gather = getattr(model, "gather_for_checkpoint", None)
    tree = gather(save_only_lora_params) if gather else layout.model_to_tree(model, save_only_lora_params)
    items["model_params"] = _snapshot(tree, rank)
    if optimizer is not None:
      shards = getattr(optimizer, "checkpoint_shards", lambda: None)()
      if shards is not None:
        otree, extras["optimizer_state"] = shards
      else:
        ogather = getattr(optimizer, "gather_for_checkpoint", None)
        otree = ogather() if ogather else layout.opt_state_to_tree(optimizer.opt_state)
      items["optimizer_state"] = _snapshot(otree, rank)
    self._last_saved_step, self._last_save_time = step, time.time()
    if self._options.enable_async_checkpointing:
      self._pending = self._executor.submit(self._write, step, items, extras, custom_metadata, init_ns, rank, world)
    else:
      self._write(step, items, extras, custom_metadata, init_ns, rank, world)
    return True

  # ---- restore -----------------------------------------------------------------------------
  def maybe_restore(self, model: torch.nn.Module, optimizer: Any = None, step: Optional[int] = None,
                    restore_only_lora_params: bool = False) -> Tuple[int, Any]:
    """Restores the latest (or the given) step into `model` / `optimizer` in place.
    Returns `(step, custom_metadata)`; `(0, {})` when there is nothing to restore."""
    t0 = time.time()
    if not self._root:
      return 0, {}
    if step is None:
      step = self.latest_step()
      if step is None:
        return 0, {}
    step_dir = os.path.join(self._root, str(step))
    md = orbax_layout.read_checkpoint_metadata(step_dir)
    mdir = os.path.join(step_dir, "model_params")
    want = layout.expected_keys(model, restore_only_lora_params)
    try:
      tree = orbax_layout.read_tree(mdir, want, partial=False)
    except KeyError as e:
      if not restore_only_lora_params:
        raise ValueError(f"Failed to restore from step {step}. If this checkpoint only contains LoRA parameters, "
                         "please set `restore_only_lora_params=True`.") from e
      raise
    scatter = getattr(model, "scatter_from_checkpoint", None)
    if scatter:
      scatter(tree, restore_only_lora_params)
    else:
      layout.tree_to_model(model, tree, restore_only_lora_params)
    odir = os.path.join(step_dir, "optimizer_state")
    index_path = os.path.join(odir, "_flat_index.json")
    if optimizer is not None and os.path.isfile(index_path) and hasattr(optimizer, "restore_shards"):
      # flat sharded state: every rank reads only the range of each array that it owns
      import json
      with open(index_path) as f:
        index = json.load(f)
      kv = orbax_layout.open_kv(odir)
      tree_md = orbax_layout.read_tree_metadata(odir)
      small = orbax_layout.read_tree(odir, [k for k in tree_md if k[0] in ("count", "hyperparams")])
      optimizer.restore_shards(index, lambda name, lo, hi: orbax_layout.read_array_rows(kv, name + ".value", lo, hi),
                               small)
    elif optimizer is not None and os.path.isdir(odir):
      otree = orbax_layout.read_tree(odir)
      oscatter = getattr(optimizer, "scatter_from_checkpoint", None)
      if oscatter:
        oscatter(otree)
      else:
        layout.tree_to_opt_state(optimizer.opt_state, otree)
    log.info("Restored params from step: %d in %.3f seconds", step, time.time() - t0)
    return step, md.get("custom_metadata", {}) or {}

  def close(self) -> None:
    if not self._root:
      return
    self.wait_until_finished()
    if self._executor is not None:
      self._executor.shutdown(wait=True)
      self._executor = None
