"""Capture of intermediate activations by module class.

Role of tunix/distillation/feature_extraction/sowed_module.py:21-179. The reference swaps
sub-modules for wrappers that `sow` their output into the module state; here a forward hook
on every sub-module of the requested classes appends its output to a list kept on the root
model, in call order. Outputs keep their autograd graph (the student's features are trained
through); the caller detaches teacher features.
"""
from __future__ import annotations

from typing import Any, Dict, List, Sequence, Type

import torch

_STATE = "_sowed_state"


def _first_tensor(out: Any) -> torch.Tensor:
  if isinstance(out, torch.Tensor):
    return out
  if isinstance(out, (tuple, list)):
    for o in out:
      if isinstance(o, torch.Tensor):
        return o
  raise TypeError(f"captured module returned no tensor: {type(out)}")


def wrap_model_with_sowed_modules(model: torch.nn.Module, modules_to_capture: Sequence[Type[torch.nn.Module]]) -> None:
  """Hooks every sub-module whose class is in `modules_to_capture` (in place)."""
  if getattr(model, _STATE, None) is not None:
    unwrap_sowed_modules(model)
  state: Dict[str, Any] = {"handles": [], "outputs": {}}
  classes = tuple(modules_to_capture)
  for name, mod in model.named_modules():
    if mod is model or not isinstance(mod, classes):
      continue

    def hook(_m, _inp, out, _name=name):
      state["outputs"].setdefault(_name, []).append(_first_tensor(out))
    state["handles"].append(mod.register_forward_hook(hook))
  if not state["handles"]:
    raise ValueError(f"no sub-module of type {[c.__name__ for c in classes]} found to capture")
  object.__setattr__(model, _STATE, state)


def pop_sowed_intermediate_outputs(model: torch.nn.Module) -> Dict[str, torch.Tensor]:
  """Returns {module path: last captured output} in registration order and clears the store."""
  state = getattr(model, _STATE, None)
  if state is None:
    raise ValueError("model has no capture hooks; call wrap_model_with_sowed_modules first")
  out = {k: v[-1] for k, v in state["outputs"].items()}
  state["outputs"].clear()
  return out


def stack_features(feats: Dict[str, torch.Tensor]) -> torch.Tensor:
  return torch.stack(list(feats.values()))


def unwrap_sowed_modules(model: torch.nn.Module) -> None:
  state = getattr(model, _STATE, None)
  if state is None:
    return
  for h in state["handles"]:
    h.remove()
  object.__setattr__(model, _STATE, None)
