"""Optimizers and learning-rate schedules with an optax-shaped surface.

Configs of the reference name optax symbols (`opt_type: adamw`, `schedule_type:
warmup_cosine_decay_schedule`, `optax.chain(optax.clip_by_global_norm(..), ..)`,
`inject_hyperparams`; tunix/cli/config.py:546-676), so the same names exist here. The
implementation is PyTorch-native: a `GradientTransformation` owns a state tree
(`count`, `mu`, `nu`, `hyperparams.learning_rate` - the same leaf names optax would
checkpoint) and updates parameters in place. bf16 parameters get an fp32 master copy; when
parameters and fp32 gradients live in flat CUDA buffers the AdamW update is one fused kernel.
"""
from __future__ import annotations

import dataclasses
import inspect
import math
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple, Union

import torch

Schedule = Callable[[int], float]
ScalarOrSchedule = Union[float, Schedule]


# ------------------------------------------------------------------------------ schedules
def constant_schedule(value: float) -> Schedule:
  return lambda count: float(value)


def polynomial_schedule(init_value: float, end_value: float, power: float, transition_steps: int,
                        transition_begin: int = 0) -> Schedule:
  def fn(count):
    if transition_steps <= 0:
      return float(init_value)
    c = min(max(count - transition_begin, 0), transition_steps)
    frac = 1 - c / transition_steps
    return float((init_value - end_value) * (frac ** power) + end_value)
  return fn


def linear_schedule(init_value: float, end_value: float, transition_steps: int, transition_begin: int = 0) -> Schedule:
  return polynomial_schedule(init_value, end_value, 1, transition_steps, transition_begin)


def cosine_decay_schedule(init_value: float, decay_steps: int, alpha: float = 0.0, exponent: float = 1.0) -> Schedule:
  def fn(count):
    if decay_steps <= 0:
      return float(init_value)
    c = min(count, decay_steps)
    cosine = 0.5 * (1 + math.cos(math.pi * c / decay_steps))
    return float(init_value * ((1 - alpha) * cosine ** exponent + alpha))
  return fn


def exponential_decay(init_value: float, transition_steps: int, decay_rate: float, transition_begin: int = 0,
                      staircase: bool = False, end_value: Optional[float] = None) -> Schedule:
  def fn(count):
    c = count - transition_begin
    if c <= 0:
      return float(init_value)
    p = c / transition_steps
    if staircase:
      p = math.floor(p)
    v = init_value * (decay_rate ** p)
    if end_value is not None:
      v = max(v, end_value) if decay_rate < 1 else min(v, end_value)
    return float(v)
  return fn


def join_schedules(schedules: Sequence[Schedule], boundaries: Sequence[int]) -> Schedule:
  def fn(count):
    idx, start = 0, 0
    for i, b in enumerate(boundaries):
      if count >= b:
        idx, start = i + 1, b
    return schedules[idx](count - start)
  return fn


def piecewise_constant_schedule(init_value: float, boundaries_and_scales: Optional[Dict[int, float]] = None) -> Schedule:
  bs = sorted((boundaries_and_scales or {}).items())
  def fn(count):
    v = init_value
    for b, s in bs:
      if count >= b:
        v *= s
    return float(v)
  return fn


def warmup_constant_schedule(init_value: float, peak_value: float, warmup_steps: int) -> Schedule:
  return join_schedules([linear_schedule(init_value, peak_value, warmup_steps), constant_schedule(peak_value)],
                        [warmup_steps])


def warmup_cosine_decay_schedule(init_value: float, peak_value: float, warmup_steps: int, decay_steps: int,
                                 end_value: float = 0.0, exponent: float = 1.0) -> Schedule:
  """Linear warm-up to `peak_value`, then cosine decay to `end_value`; `decay_steps` counts
  from step 0 (it includes the warm-up), as in optax."""
  alpha = 0.0 if peak_value == 0.0 else end_value / peak_value
  return join_schedules([
      linear_schedule(init_value, peak_value, warmup_steps),
      cosine_decay_schedule(peak_value, max(decay_steps - warmup_steps, 0), alpha, exponent),
  ], [warmup_steps])


def warmup_exponential_decay_schedule(init_value: float, peak_value: float, warmup_steps: int, transition_steps: int,
                                      decay_rate: float, transition_begin: int = 0, staircase: bool = False,
                                      end_value: Optional[float] = None) -> Schedule:
  return join_schedules([
      linear_schedule(init_value, peak_value, warmup_steps),
      exponential_decay(peak_value, transition_steps, decay_rate, transition_begin, staircase, end_value),
  ], [warmup_steps])


class _Schedules:
  """`optim.schedules.<name>` namespace (mirrors `optax.schedules`)."""
  constant_schedule = staticmethod(constant_schedule)
  polynomial_schedule = staticmethod(polynomial_schedule)
  linear_schedule = staticmethod(linear_schedule)
  cosine_decay_schedule = staticmethod(cosine_decay_schedule)
  exponential_decay = staticmethod(exponential_decay)
  join_schedules = staticmethod(join_schedules)
  piecewise_constant_schedule = staticmethod(piecewise_constant_schedule)
  warmup_constant_schedule = staticmethod(warmup_constant_schedule)
  warmup_cosine_decay_schedule = staticmethod(warmup_cosine_decay_schedule)
  warmup_exponential_decay_schedule = staticmethod(warmup_exponential_decay_schedule)

  @staticmethod
  def inject_hyperparams(factory):
    return inject_hyperparams(factory)


schedules = _Schedules()


def _lr_at(lr: ScalarOrSchedule, count: int) -> float:
  return float(lr(count)) if callable(lr) else float(lr)


# ------------------------------------------------------------------------------ transformations
Params = Dict[str, torch.Tensor]


class GradientTransformation:
  """Base class. `init` builds the state tree; `apply` updates `params` in place from `grads`.

  `grads[name]` may be fp32 while `params[name]` is bf16 (gradient accumulation buffers).
  `grad_scale` multiplies every gradient first (1/denominator, clipping); it may be a Python
  float or a 0-d device tensor (no host sync).
  """

  exposes_hyperparams = False

  def init(self, params: Params) -> Dict[str, Any]:
    return {}

  def apply(self, params: Params, grads: Params, state: Dict[str, Any], grad_scale: Any = None) -> None:
    raise NotImplementedError

  def learning_rate(self, state: Dict[str, Any]) -> Optional[float]:
    return None

  # clipping transforms report the max norm so a trainer can fold it into `grad_scale`
  max_grad_norm: Optional[float] = None


def _scaled(g: torch.Tensor, grad_scale: Any) -> torch.Tensor:
  g = g.float() if g.dtype != torch.float32 else g
  if grad_scale is None:
    return g
  return g * grad_scale


def _needs_master(p: torch.Tensor) -> bool:
  return p.dtype in (torch.bfloat16, torch.float16)


class _MomentOptimizer(GradientTransformation):
  """Shared plumbing for sgd/adam-family optimizers: step counter, fp32 master copies of
  low-precision parameters, per-parameter update with decoupled weight decay."""

  def __init__(self, learning_rate: ScalarOrSchedule, weight_decay: float = 0.0,
               mask: Optional[Callable[[str, torch.Tensor], bool]] = None, expose_hyperparams: bool = False):
    self._lr = learning_rate
    self.weight_decay = weight_decay
    self._mask = mask
    self.exposes_hyperparams = expose_hyperparams

  def _base_state(self, params: Params) -> Dict[str, Any]:
    st: Dict[str, Any] = {"count": torch.zeros((), dtype=torch.int32)}
    master = {n: p.detach().float().clone() for n, p in params.items() if _needs_master(p)}
    if master:
      st["master"] = master
    if self.exposes_hyperparams:
      st["hyperparams"] = {"learning_rate": torch.tensor(_lr_at(self._lr, 0), dtype=torch.float32)}
    return st

  def learning_rate(self, state):
    return _lr_at(self._lr, int(state["count"]))

  def _decay(self, name: str, p: torch.Tensor) -> float:
    if self.weight_decay == 0.0:
      return 0.0
    if self._mask is not None and not self._mask(name, p):
      return 0.0
    return self.weight_decay

  def _direction(self, name: str, g: torch.Tensor, state: Dict[str, Any], count: int) -> torch.Tensor:
    raise NotImplementedError

  @torch.no_grad()
  def apply(self, params, grads, state, grad_scale=None):
    count = int(state["count"]) + 1
    lr = _lr_at(self._lr, count - 1)
    masters = state.get("master", {})
    for name, p in params.items():
      g = grads.get(name)
      if g is None:
        continue
      g = _scaled(g, grad_scale)
      w = masters.get(name, p)
      d = self._direction(name, g, state, count)
      wd = self._decay(name, p)
      if wd:
        d = d + wd * w
      w.add_(d.to(w.dtype), alpha=-lr)
      if w is not p:
        p.copy_(w)
    state["count"] = torch.tensor(count, dtype=torch.int32)
    if "hyperparams" in state:
      state["hyperparams"]["learning_rate"] = torch.tensor(_lr_at(self._lr, count), dtype=torch.float32)


class _SGD(_MomentOptimizer):

  def __init__(self, learning_rate, momentum: Optional[float] = None, nesterov: bool = False, **kw):
    super().__init__(learning_rate, **kw)
    self.momentum, self.nesterov = momentum, nesterov

  def init(self, params):
    st = self._base_state(params)
    if self.momentum:
      st["trace"] = {n: torch.zeros_like(p, dtype=torch.float32 if _needs_master(p) else p.dtype)
                     for n, p in params.items()}
    return st

  def _direction(self, name, g, state, count):
    if not self.momentum:
      return g
    t = state["trace"][name]
    t.mul_(self.momentum).add_(g.to(t.dtype))
    return (g + self.momentum * t) if self.nesterov else t


class _Adam(_MomentOptimizer):

  def __init__(self, learning_rate, b1=0.9, b2=0.999, eps=1e-8, eps_root=0.0, mu_dtype=None, **kw):
    super().__init__(learning_rate, **kw)
    self.b1, self.b2, self.eps, self.eps_root, self.mu_dtype = b1, b2, eps, eps_root, mu_dtype

  def init(self, params):
    st = self._base_state(params)
    # Moments follow the parameter dtype (fp32 for parameters that carry an fp32 master copy),
    # which is what zeros_like(params) gives in the reference (tunix/sft/peft_trainer.py:174-198).
    def mdt(p):
      if self.mu_dtype is not None:
        return self.mu_dtype
      return torch.float32 if _needs_master(p) else p.dtype
    st["mu"] = {n: torch.zeros_like(p, dtype=mdt(p)) for n, p in params.items()}
    st["nu"] = {n: torch.zeros_like(p, dtype=torch.float32 if _needs_master(p) else p.dtype)
                for n, p in params.items()}
    return st

  def _direction(self, name, g, state, count):
    mu, nu = state["mu"][name], state["nu"][name]
    mu.mul_(self.b1).add_(g.to(mu.dtype), alpha=1 - self.b1)
    nu.mul_(self.b2).addcmul_(g.to(nu.dtype), g.to(nu.dtype), value=1 - self.b2)
    mhat = mu.float() / (1 - self.b1 ** count)
    vhat = nu.float() / (1 - self.b2 ** count)
    return mhat / (torch.sqrt(vhat + self.eps_root) + self.eps)

  @torch.no_grad()
  def apply(self, params, grads, state, grad_scale=None):
    """CUDA parameters with an fp32 master copy take the fused kernel (one pass over master,
    moments and gradient, no temporaries); everything else takes the generic path."""
    masters = state.get("master", {})
    fused = [n for n, p in params.items()
             if p.is_cuda and n in masters and grads.get(n) is not None and grads[n].dtype == torch.float32
             and grads[n].is_contiguous() and self.fusable and state["mu"][n].dtype == torch.float32]
    if not fused:
      return super().apply(params, grads, state, grad_scale)
    from .ops import kernels
    count = int(state["count"]) + 1
    lr = _lr_at(self._lr, count - 1)
    dev = params[fused[0]].device
    gs = grad_scale
    if gs is not None and not isinstance(gs, torch.Tensor):
      gs = torch.tensor([float(gs)], dtype=torch.float32, device=dev)
    elif gs is not None:
      gs = gs.reshape(1).to(torch.float32)
    for n in fused:
      kernels.adamw_step(masters[n], state["mu"][n], state["nu"][n], grads[n], params[n], lr=lr, beta1=self.b1,
                         beta2=self.b2, eps=self.eps, weight_decay=self.weight_decay, step=count, grad_scale=gs,
                         zero_grad=False)
    rest = {n: p for n, p in params.items() if n not in set(fused)}
    if rest:
      saved = state["count"]
      super().apply(rest, grads, state, grad_scale)
      state["count"] = saved
    state["count"] = torch.tensor(count, dtype=torch.int32)
    if "hyperparams" in state:
      state["hyperparams"]["learning_rate"] = torch.tensor(_lr_at(self._lr, count), dtype=torch.float32)

  # ---- fused flat path --------------------------------------------------------------
  def fused_flat_step(self, flat_master, flat_mu, flat_nu, flat_grad, flat_param_bf16, state, grad_scale,
                      zero_grad=True) -> None:
    """One-kernel AdamW over flat fp32 buffers (CUDA). `grad_scale` is a device scalar or None."""
    from .ops import kernels
    count = int(state["count"]) + 1
    lr = _lr_at(self._lr, count - 1)
    gs = grad_scale
    if gs is not None and not isinstance(gs, torch.Tensor):
      gs = torch.tensor([float(gs)], dtype=torch.float32, device=flat_master.device)
    kernels.adamw_step(flat_master, flat_mu, flat_nu, flat_grad, flat_param_bf16, lr=lr, beta1=self.b1,
                       beta2=self.b2, eps=self.eps, weight_decay=self.weight_decay, step=count, grad_scale=gs,
                       zero_grad=zero_grad)
    state["count"] = torch.tensor(count, dtype=torch.int32)
    if "hyperparams" in state:
      state["hyperparams"]["learning_rate"] = torch.tensor(_lr_at(self._lr, count), dtype=torch.float32)

  @property
  def fusable(self) -> bool:
    return self._mask is None and self.eps_root == 0.0 and self.mu_dtype in (None, torch.float32)


class _Lion(_MomentOptimizer):

  def __init__(self, learning_rate, b1=0.9, b2=0.99, **kw):
    super().__init__(learning_rate, **kw)
    self.b1, self.b2 = b1, b2

  def init(self, params):
    st = self._base_state(params)
    st["mu"] = {n: torch.zeros_like(p, dtype=torch.float32 if _needs_master(p) else p.dtype) for n, p in params.items()}
    return st

  def _direction(self, name, g, state, count):
    mu = state["mu"][name]
    d = torch.sign(self.b1 * mu + (1 - self.b1) * g.to(mu.dtype))
    mu.mul_(self.b2).add_(g.to(mu.dtype), alpha=1 - self.b2)
    return d


class _RMSProp(_MomentOptimizer):

  def __init__(self, learning_rate, decay=0.9, eps=1e-8, **kw):
    super().__init__(learning_rate, **kw)
    self.decay, self.eps = decay, eps

  def init(self, params):
    st = self._base_state(params)
    st["nu"] = {n: torch.zeros_like(p, dtype=torch.float32 if _needs_master(p) else p.dtype) for n, p in params.items()}
    return st

  def _direction(self, name, g, state, count):
    nu = state["nu"][name]
    nu.mul_(self.decay).addcmul_(g.to(nu.dtype), g.to(nu.dtype), value=1 - self.decay)
    return g / (torch.sqrt(nu.float()) + self.eps)


class _Adagrad(_MomentOptimizer):

  def __init__(self, learning_rate, initial_accumulator_value=0.1, eps=1e-7, **kw):
    super().__init__(learning_rate, **kw)
    self.init_acc, self.eps = initial_accumulator_value, eps

  def init(self, params):
    st = self._base_state(params)
    st["sum_of_squares"] = {n: torch.full_like(p, self.init_acc, dtype=torch.float32) for n, p in params.items()}
    return st

  def _direction(self, name, g, state, count):
    acc = state["sum_of_squares"][name]
    acc.addcmul_(g, g)
    return g / (torch.sqrt(acc) + self.eps)


def sgd(learning_rate: ScalarOrSchedule, momentum: Optional[float] = None, nesterov: bool = False):
  return _SGD(learning_rate, momentum, nesterov)


def adam(learning_rate: ScalarOrSchedule, b1=0.9, b2=0.999, eps=1e-8, eps_root=0.0, mu_dtype=None):
  return _Adam(learning_rate, b1, b2, eps, eps_root, mu_dtype)


def adamw(learning_rate: ScalarOrSchedule, b1=0.9, b2=0.999, eps=1e-8, eps_root=0.0, mu_dtype=None,
          weight_decay: float = 1e-4, mask=None):
  return _Adam(learning_rate, b1, b2, eps, eps_root, mu_dtype, weight_decay=weight_decay, mask=mask)


def lion(learning_rate: ScalarOrSchedule, b1=0.9, b2=0.99, weight_decay: float = 1e-3, mask=None):
  return _Lion(learning_rate, b1, b2, weight_decay=weight_decay, mask=mask)


def rmsprop(learning_rate: ScalarOrSchedule, decay=0.9, eps=1e-8):
  return _RMSProp(learning_rate, decay, eps)


def adagrad(learning_rate: ScalarOrSchedule, initial_accumulator_value=0.1, eps=1e-7):
  return _Adagrad(learning_rate, initial_accumulator_value, eps)


class _ClipByGlobalNorm(GradientTransformation):

  def __init__(self, max_norm: float):
    self.max_grad_norm = float(max_norm)


def clip_by_global_norm(max_norm: float) -> GradientTransformation:
  """Marker transformation: the trainer computes the fp32 global norm once and folds
  `min(1, max_norm / norm)` into the gradient scale handed to the optimizer."""
  return _ClipByGlobalNorm(max_norm)


def global_norm(grads: Params) -> torch.Tensor:
  """fp32 L2 norm over all tensors."""
  tensors = [g for g in grads.values() if g is not None]
  if not tensors:
    return torch.zeros(())
  sq = torch.stack([g.float().pow(2).sum() for g in tensors])
  return torch.sqrt(sq.sum())


class _Chain(GradientTransformation):

  def __init__(self, parts: Sequence[GradientTransformation]):
    self.parts = list(parts)
    self.inner = None
    for p in self.parts:
      if isinstance(p, _ClipByGlobalNorm):
        self.max_grad_norm = p.max_grad_norm
      elif self.inner is None:
        self.inner = p
      else:
        raise ValueError("chain() supports clip_by_global_norm plus exactly one optimizer")
    if self.inner is None:
      raise ValueError("chain() needs an optimizer")
    self.exposes_hyperparams = self.inner.exposes_hyperparams

  def init(self, params):
    return self.inner.init(params)

  def apply(self, params, grads, state, grad_scale=None):
    self.inner.apply(params, grads, state, grad_scale)

  def learning_rate(self, state):
    return self.inner.learning_rate(state)

  def __getattr__(self, item):  # fused path / hyperparameters live on the inner optimizer
    if item in ("parts", "inner"):
      raise AttributeError(item)
    return getattr(self.inner, item)


def chain(*parts: GradientTransformation) -> GradientTransformation:
  return _Chain(parts)


def inject_hyperparams(factory: Callable[..., GradientTransformation]):
  """`inject_hyperparams(adamw)(learning_rate=schedule, ...)`: the state tree then carries
  `hyperparams.learning_rate`, which the trainer logs every step."""
  def make(*args, **kwargs):
    tx = factory(*args, **kwargs)
    inner = tx.inner if isinstance(tx, _Chain) else tx
    inner.exposes_hyperparams = True
    tx.exposes_hyperparams = True
    return tx
  return make


_FACTORIES = {
    "sgd": sgd, "adam": adam, "adamw": adamw, "lion": lion, "rmsprop": rmsprop, "adagrad": adagrad,
}


def get_optimizer_factory(name: str) -> Callable[..., GradientTransformation]:
  if name not in _FACTORIES:
    raise ValueError(f"Unknown optimizer {name!r}; available: {sorted(_FACTORIES)}")
  return _FACTORIES[name]


def get_schedule_factory(name: str) -> Callable[..., Schedule]:
  fn = getattr(schedules, name, None)
  if fn is None or name == "inject_hyperparams":
    raise ValueError(f"Unknown schedule {name!r}")
  return fn


def filter_kwargs(fn: Callable, kwargs: Dict[str, Any]) -> Dict[str, Any]:
  """Keeps the entries of `kwargs` that `fn` accepts (configs carry a superset of options)."""
  sig = inspect.signature(fn)
  return {k: v for k, v in kwargs.items() if k in sig.parameters and v is not None}
