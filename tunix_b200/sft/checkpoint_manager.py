"""Checkpoint manager: policy-driven, asynchronous saves and restore-on-construction.

API and semantics follow tunix/sft/checkpoint_manager.py:98-331: checkpointables `model_params`
(+ `optimizer_state`), LoRA-only save / partial restore, custom metadata, `maybe_restore`
returning `(step, custom_metadata)`. Files are written in the Orbax directory layout
(`tunix_b200.ckpt.orbax_layout`).

A save first snapshots the tensors to host memory on the calling thread (so training may
overwrite the GPU copies immediately), then a background thread writes the files into
`<root>/<step>.tmp-*` and renames the directory into place - a step directory exists only
when complete. In multi-rank jobs rank 0 of the model's mesh writes replicated state; sharded
state is gathered by `tunix_b200.dist` before it reaches this class.
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


def _rank() -> int:
  return int(os.environ.get("RANK", "0"))


def _snapshot(tree: Mapping[Any, torch.Tensor]) -> Dict[Any, torch.Tensor]:
  """Device -> host copy of every leaf (pinned staging for CUDA tensors)."""
  out = {}
  for k, t in tree.items():
    t = torch.as_tensor(t).detach()
    if t.is_cuda:
      host = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=True)
      host.copy_(t, non_blocking=True)
      out[k] = host
    else:
      out[k] = t.clone()
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
  def _write(self, step: int, items: Dict[str, Dict[Any, torch.Tensor]], custom_metadata, init_ns: int) -> None:
    final = os.path.join(self._root, str(step))
    tmp = f"{final}.tmp-{os.getpid()}-{init_ns}"
    try:
      for name, tree in items.items():
        orbax_layout.write_tree(os.path.join(tmp, name), tree)
      orbax_layout.write_checkpoint_metadata(tmp, list(items.keys()), custom_metadata, init_ns)
      if os.path.exists(final):
        shutil.rmtree(final)
      os.replace(tmp, final)
    finally:
      if os.path.exists(tmp):
        shutil.rmtree(tmp, ignore_errors=True)
    policy = self._options.preservation_policy
    if policy is not None:
      for s in policy.to_delete(orbax_layout.list_steps(self._root)):
        shutil.rmtree(os.path.join(self._root, str(s)), ignore_errors=True)

  def save(self, step: int, model: torch.nn.Module, optimizer: Any = None, save_only_lora_params: bool = False,
           force: bool = False, custom_metadata: Optional[Mapping[str, Any]] = None) -> bool:
    """Saves the parameters (and optimizer state) for `step`. Returns whether a save was
    performed (synchronous mode) or started (asynchronous mode)."""
    if not self._root:
      return False
    if not force:
      if self._pending is not None and not self._pending.done():
        return False    # a save is still being written; the continuous policy skips this step
      if not self._options.save_decision_policy.should_save(step, self._last_saved_step, self._last_save_time):
        return False
    if self._last_saved_step == step:
      return False
    self.wait_until_finished()
    init_ns = time.time_ns()
    items: Dict[str, Dict[Any, torch.Tensor]] = {}
    gather = getattr(model, "gather_for_checkpoint", None)
    tree = gather(save_only_lora_params) if gather else layout.model_to_tree(model, save_only_lora_params)
    if optimizer is not None:
      ogather = getattr(optimizer, "gather_for_checkpoint", None)
      otree = ogather() if ogather else layout.opt_state_to_tree(optimizer.opt_state)
    if _rank() != 0:
      self._last_saved_step, self._last_save_time = step, time.time()
      return True
    items["model_params"] = _snapshot(tree)
    if optimizer is not None:
      items["optimizer_state"] = _snapshot(otree)
    self._last_saved_step, self._last_save_time = step, time.time()
    if self._options.enable_async_checkpointing:
      self._pending = self._executor.submit(self._write, step, items, custom_metadata, init_ns)
    else:
      self._write(step, items, custom_metadata, init_ns)
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
    if optimizer is not None and os.path.isdir(odir):
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
