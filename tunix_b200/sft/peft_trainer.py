"""Generic trainer for full-weight and LoRA fine-tuning.

Behaviour follows tunix/sft/peft_trainer.py:321-1263: gradients are taken of the *unreduced*
loss sum and divided by the summed denominators of all micro-batches of an update (global
weighted mean, not a mean of means); the fp32 global gradient norm is logged every step (0 on
accumulation-only steps); metrics are written one step late so host I/O overlaps the next step;
checkpoints restore on construction and the data iterator is fast-forwarded on resume.

Execution differs by design: there is no tracing compiler. A step is eager PyTorch whose hot
ops are sm_100a kernels; weight gradients are accumulated in fp32 straight from the GEMM
epilogues into `main_grad` buffers; the host never waits for the device inside a step (loss
and norm stay on the GPU until the metrics of the *previous* step are written).
"""
from __future__ import annotations

import contextlib
import dataclasses
import logging
import time
from typing import Any, Callable, Dict, Iterable, List, Mapping, Optional, Tuple

import numpy as np
import torch

from ..common.configs import TrainingConfig
from .. import optim as optim_lib
from . import checkpoint_manager as ckpt_lib
from . import hooks as hooks_lib
from . import inflight_throttler, metrics_logger as ml, profiler, progress_bar, sharding_utils, utils
from .metrics_logger import MetricsLogger, Mode

log = logging.getLogger(__name__)

LossOutput = utils.LossOutput
WeightedMetric = utils.WeightedMetric


@dataclasses.dataclass
class TrainingInput:
  """A batch of token ids `[B, L]` and its loss mask `[B, L]` (1 = contributes to the loss)."""

  input_tokens: Any
  input_mask: Any
  images: Any = None


def _to_float(v: Any) -> float:
  if isinstance(v, torch.Tensor):
    return float(v.detach().float().item())
  return float(np.asarray(v, dtype=np.float64))


def _weighted_metric_mean(values: Iterable[Any]) -> float:
  """Global weighted mean over WeightedMetrics: sum(sums) / sum(denominators)."""
  values = list(values)
  total = sum(_to_float(v.unreduced_sum) for v in values)
  denom = sum(_to_float(v.denominator) for v in values)
  first = values[0]
  return _to_float(WeightedMetric(total, denom, first.eps, first.min_denom).compute())


def _metric_reducer(metric: Any) -> Callable[[Any], Any]:
  return _weighted_metric_mean if isinstance(metric, WeightedMetric) else np.mean


@dataclasses.dataclass
class MetricsBuffer:
  """Losses and metrics of the micro-steps of one optimizer step."""

  step: int
  losses: List[Any]
  additional_metrics: Dict[str, Tuple[List[Any], Callable]] = dataclasses.field(default_factory=dict)

  @property
  def loss(self):
    if isinstance(self.losses[0], WeightedMetric):
      return _weighted_metric_mean(self.losses)
    return float(np.mean([_to_float(l) for l in self.losses]))


class GradientAccumulator:
  """fp32 accumulation buffers for the trainable parameters plus the scalar denominator.

  CUDA bf16 parameters expose their buffer as `param.main_grad`, which the kernel backward
  passes add into directly; gradients that arrive through `param.grad` (CPU path, ops without
  a fused epilogue) are folded in by `collect()`. `get_scale()` is the zero-safe
  1 / sum(denominators) as a device scalar.
  """

  def __init__(self, named_params: Mapping[str, torch.nn.Parameter]):
    self.params = dict(named_params)
    self.acc: Dict[str, torch.Tensor] = {}
    dev = None
    for n, p in self.params.items():
      dev = p.device
      if getattr(p, "grad_managed", False):
        continue                      # a sharded-parameter store collects and reduces this gradient itself
      buf = getattr(p, "main_grad", None)
      if buf is None:
        buf = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
        if p.is_cuda and p.dtype == torch.bfloat16:
          p.main_grad = buf
      self.acc[n] = buf
      dev = p.device
    self.denom = torch.zeros((), dtype=torch.float32, device=dev or "cpu")

  def collect(self, denom: Any) -> None:
    for n, buf in self.acc.items():
      p = self.params[n]
      if p.grad is not None:
        buf.add_(p.grad.to(torch.float32))
        p.grad = None
    if isinstance(denom, torch.Tensor):
      self.denom.add_(denom.detach().to(self.denom.device, torch.float32))
    else:
      self.denom.add_(float(denom))

  def get_scale(self) -> torch.Tensor:
    d = self.denom
    return torch.where(d == 0, torch.zeros_like(d), 1.0 / torch.where(d == 0, torch.ones_like(d), d))

  def reset(self, zero_grads: bool = True) -> None:
    if zero_grads:
      for b in self.acc.values():
        b.zero_()
    self.denom.zero_()


class ModelOptimizer:
  """Binds a `GradientTransformation` to the trainable parameters of a model (the role
  `nnx.Optimizer(model, tx, wrt=...)` plays in the reference). When the model carries a
  `flat_store` (`tunix_b200.dist.fsdp.shard_model`) the optimizer state is flat and sharded
  and the update is the store's fused step."""

  def __init__(self, model: torch.nn.Module, tx: optim_lib.GradientTransformation, lora_only: bool):
    self.tx = tx
    if lora_only:
      for n, p in model.named_parameters():
        if not getattr(p, "is_lora", False):
          p.requires_grad_(False)
    self.named_params = {n: p for n, p in model.named_parameters()
                         if p.requires_grad and (getattr(p, "is_lora", False) or not lora_only)}
    self.flat = getattr(model, "flat_store", None)
    inner = getattr(tx, "inner", tx)
    if self.flat is not None and not (hasattr(inner, "fused_flat_step") and inner.fusable):
      raise ValueError("a flat parameter store needs an Adam-family optimizer without mask/eps_root")
    self.opt_state = self.flat.init_state(tx) if self.flat is not None else tx.init(self.named_params)

  def update(self, grads: Mapping[str, torch.Tensor], grad_scale: Any = None) -> None:
    self.tx.apply(self.named_params, grads, self.opt_state, grad_scale)

  @property
  def step(self) -> int:
    return int(self.opt_state.get("count", 0))

  def learning_rate(self) -> Optional[float]:
    hp = self.opt_state.get("hyperparams")
    if hp is not None and "learning_rate" in hp:
      return _to_float(hp["learning_rate"])
    return None

  # checkpoint hooks used by CheckpointManager
  def checkpoint_group(self):
    """Process group whose ranks save and restore together (None: a single process)."""
    return self.flat.group if self.flat is not None and self.flat.world > 1 else None

  def checkpoint_shards(self):
    """(tree, extras) when the state is sharded over ranks: every rank contributes its own chunks and no
    state is gathered. None for single-rank state, which is saved per parameter."""
    if self.flat is None or self.flat.world == 1:
      return None
    import json
    return self.flat.state_shards(self.opt_state), {"_flat_index.json": json.dumps(self.flat.flat_index()).encode()}

  def restore_shards(self, index, read_rows, small: Mapping[Any, torch.Tensor]) -> None:
    """Inverse of `checkpoint_shards`: `read_rows(name, lo, hi)` reads a range of a flat array, `small`
    holds the replicated leaves (step count, hyper-parameters)."""
    self.flat.load_state_shards(self.opt_state, index, read_rows)
    if ("count", "value") in small:
      self.opt_state["count"] = small[("count", "value")].to(torch.int32).reshape(())
    for key, v in small.items():
      if key[0] == "hyperparams" and "hyperparams" in self.opt_state:
        self.opt_state["hyperparams"][key[1]] = v.to(torch.float32).reshape(())
    self._master_restored = True

  def gather_for_checkpoint(self):
    from ..ckpt import layout
    st = self.flat.opt_state_tree(self.opt_state) if self.flat is not None else self.opt_state
    return layout.opt_state_to_tree(st)

  def scatter_from_checkpoint(self, tree) -> None:
    from ..ckpt import layout
    if self.flat is None:
      layout.tree_to_opt_state(self.opt_state, tree)
      return
    shadow = {k: ({n: torch.zeros(self.flat.shapes[n], dtype=torch.float32) for n in self.flat.names}
                  if k in ("mu", "nu", "master") else v) for k, v in self.opt_state.items()}
    layout.tree_to_opt_state(shadow, tree)
    self.flat.load_opt_state_tree(self.opt_state, shadow)
    if "hyperparams" in shadow and "hyperparams" in self.opt_state:
      self.opt_state["hyperparams"] = shadow["hyperparams"]
    self._master_restored = True

  def sync_master_if_needed(self) -> None:
    """After a restore that did not carry optimizer state the fp32 master shard is re-derived
    from the restored bf16 parameters."""
    if self.flat is not None and not getattr(self, "_master_restored", False):
      self.flat.refresh_master_from_params(self.opt_state)


class _NoopSpan:

  def device_end(self, *a, **k):
    pass

  def async_end(self, *a, **k):
    pass


class _NoopTracer:

  @contextlib.contextmanager
  def span(self, *a, **k):
    yield _NoopSpan()

  @contextlib.contextmanager
  def span_group(self, *a, **k):
    yield _NoopSpan()


class PeftTrainer:
  """Training loop for full-weight or LoRA fine-tuning; only LoRA parameters are updated
  when the model carries LoRA adapters.

  To monitor the learning rate build the optimizer with
  `optim.inject_hyperparams(optim.adamw)(learning_rate=schedule)`.
  """

  supports_sequence_packing = True

  def __init__(self, model: torch.nn.Module, optimizer: optim_lib.GradientTransformation,
               training_config: TrainingConfig, metrics_logger: Optional[MetricsLogger] = None,
               perf_tracer: Any = None, perf_tracer_v2: Any = None):
    if training_config.max_seq_token_per_tpu is not None and not self.supports_sequence_packing:
      raise ValueError("Sequence packing is not supported by this trainer.")
    self.model = model
    self.config = training_config
    self._lora_enabled = utils.is_lora_enabled(model)
    self.optimizer = ModelOptimizer(model, optimizer, lora_only=self._lora_enabled)
    self.grad_accumulator = GradientAccumulator(self.optimizer.named_params)
    self._max_grad_norm = training_config.max_grad_norm or getattr(optimizer, "max_grad_norm", None)

    self.loss_fn = _default_loss_fn
    self.eval_loss_fn = _default_loss_fn
    self.gen_model_input_fn = _default_gen_model_input_fn
    self.checkpoint_manager = ckpt_lib.CheckpointManager(root_directory=self.config.checkpoint_root_directory,
                                                         options=self.config.checkpointing_options)
    self.metrics_logger = metrics_logger or MetricsLogger(self.config.metrics_logging_options)
    self.metrics_prefix = self.config.metrics_prefix
    self.is_managed_externally = False
    self._perf_tracer = perf_tracer if perf_tracer is not None else _NoopTracer()
    self._perf_tracer_v2 = perf_tracer_v2 if perf_tracer_v2 is not None else _NoopTracer()

    self._train_steps = 0   # number of optimizer updates
    self._iter_steps = 0    # number of micro-steps
    self._throttler = inflight_throttler.InflightThrottler(training_config.max_inflight_computations)
    self._mode: Mode = Mode.TRAIN
    self._has_aux = False
    self._pbar = None

    self._train_steps, self._restored_custom_metadata = self.checkpoint_manager.maybe_restore(
        self.model, self.optimizer, restore_only_lora_params=self._lora_enabled)
    if self._train_steps > 0:
      self.optimizer.sync_master_if_needed()
    ga = self.config.get_with_default("gradient_accumulation_steps", 1)
    self._iter_steps = self._train_steps * ga
    max_step = self.config.max_steps * ga if self.config.max_steps is not None else None
    self._prof = profiler.Profiler(self._iter_steps, max_step, self.config.profiler_options)
    self._buffered_train_metrics: Optional[MetricsBuffer] = None
    self._prev_buffered_train_metrics: Optional[MetricsBuffer] = None
    self._buffered_eval_metrics: Optional[MetricsBuffer] = None
    self.training_hooks: Optional[hooks_lib.TrainingHooks] = None
    self.data_hooks: Optional[hooks_lib.DataHooks] = None
    self._mini_batch_size = None
    self._grad_sync = None   # set by tunix_b200.dist when the model is sharded/replicated
    self._zero_norm = None
    self._closing = False
    try:
      self._device = next(model.parameters()).device
    except StopIteration:
      self._device = None

  # ---- configuration ---------------------------------------------------------------
  def with_training_hooks(self, training_hooks: hooks_lib.TrainingHooks):
    self.training_hooks = training_hooks
    return self

  def with_data_hooks(self, data_hooks: hooks_lib.DataHooks):
    self.data_hooks = data_hooks
    return self

  def clear_jit_cache(self):
    """Kept for API compatibility; there is no compilation cache to clear."""

  def with_loss_fn(self, loss_fn: Callable[..., Any], has_aux: bool = False):
    self.loss_fn = loss_fn
    self.eval_loss_fn = loss_fn
    self._has_aux = has_aux
    return self

  def with_gen_model_input_fn(self, gen_model_input_fn: Callable[[Any], Dict[str, Any]]):
    """`gen_model_input_fn(batch) -> kwargs` for the loss function."""
    self.gen_model_input_fn = gen_model_input_fn
    return self

  def with_grad_sync(self, grad_sync: Any):
    """Installs the data-parallel gradient/denominator reduction (`tunix_b200.dist`)."""
    self._grad_sync = grad_sync
    return self

  # ---- one step ----------------------------------------------------------------------
  def _split_loss(self, out: Any) -> Tuple[torch.Tensor, Any, Any]:
    """-> (tensor to differentiate, aux, denominator)."""
    if isinstance(out, LossOutput):
      return out.primary_loss.unreduced_sum, out, out.primary_loss.denominator
    if self._has_aux:
      return out[0], out[1], 1.0
    return out, None, 1.0

  def _train_step(self, inputs: Any, is_update_step: bool):
    model_inputs = self.gen_model_input_fn(inputs)
    self.model.train()
    out = self.loss_fn(self.model, **model_inputs)
    loss_t, aux, denom = self._split_loss(out)
    if is_update_step and self.optimizer.flat is not None:
      self.optimizer.flat.arm_overlap()      # gradients of this backward pass are final: reduce buckets as they finish
    loss_t.backward()
    if self.optimizer.flat is not None:
      self.optimizer.flat.after_backward()
    loss_val = aux.primary_loss.compute().detach() if isinstance(aux, LossOutput) else loss_t.detach()
    acc = self.grad_accumulator
    acc.collect(denom)
    if is_update_step:
      if self._grad_sync is not None:
        self._grad_sync.reduce(acc)
      grad_norm = self._apply_update()
    else:
      if self._zero_norm is None:
        self._zero_norm = torch.zeros((), dtype=torch.float32, device=acc.denom.device)
      grad_norm = self._zero_norm
    if isinstance(aux, LossOutput):
      aux = LossOutput(aux.primary_loss.detach(),
                       {k: (v.detach() if isinstance(v, (WeightedMetric, torch.Tensor)) else v)
                        for k, v in aux.aux_metrics.items()})
    return loss_val, aux, grad_norm

  def _apply_update(self) -> torch.Tensor:
    """Scales accumulated grads by 1/sum(denom), computes the fp32 global norm, clips, steps."""
    acc = self.grad_accumulator
    scale = acc.get_scale()
    if self.optimizer.flat is not None:
      norm = self.optimizer.flat.step(self.optimizer.tx, self.optimizer.opt_state, acc.denom, self._max_grad_norm)
      acc.reset(zero_grads=False)
      return norm
    grads = acc.acc
    if all(g.is_cuda and g.is_contiguous() for g in grads.values()):
      from ..ops import kernels
      sq = torch.zeros(1, dtype=torch.float32, device=acc.denom.device)
      for g in grads.values():
        kernels.sumsq(g.view(-1), sq, accumulate=True)
      sq = sq[0]
    elif any(g.is_cuda for g in grads.values()):
      sq = torch.stack([g.pow(2).sum() for g in grads.values()]).sum()
    else:
      sq = sum(g.double().pow(2).sum() for g in grads.values()).float()
    if self._grad_sync is not None:
      sq = self._grad_sync.reduce_norm_sq(sq)
    norm = torch.sqrt(sq) * scale
    gs = scale
    if self._max_grad_norm:
      gs = scale * torch.clamp(self._max_grad_norm / (norm + 1e-6), max=1.0)
    self.optimizer.update(grads, gs)
    acc.reset()
    return norm

  @torch.no_grad()
  def _eval_step(self, inputs: Any):
    model_inputs = self.gen_model_input_fn(inputs)
    self.model.eval()
    out = self.eval_loss_fn(self.model, **model_inputs)
    if isinstance(out, LossOutput):
      return out.primary_loss.compute(), out
    if self._has_aux:
      return out[0], out[1]
    return out, None

  def create_train_step_fn(self):
    return self._train_step

  def create_eval_step_fn(self):
    return self._eval_step

  # ---- hooks for subclasses ------------------------------------------------------------
  def _prepare_inputs(self, input_data: Any) -> Any:
    return input_data

  def _post_process_train_step(self, aux: Any) -> None:
    pass

  def _post_process_eval_step(self, aux: Any) -> None:
    pass

  def _try_get_learning_rate(self) -> Optional[float]:
    return self.optimizer.learning_rate()

  # ---- metrics ---------------------------------------------------------------------------
  def _log_metrics(self, loss: Any, step: Optional[int] = None, additional_metrics: Optional[Dict[str, Any]] = None):
    loss = _to_float(loss)
    perplexity = float(np.exp(min(loss, 700.0)))
    self.metrics_logger.log(self.metrics_prefix, "loss", loss, self._mode, step)
    self.metrics_logger.log(self.metrics_prefix, "perplexity", perplexity, self._mode, step)
    lr = self._try_get_learning_rate()
    if lr is not None:
      self.metrics_logger.log(self.metrics_prefix, "learning_rate", lr, self._mode, step)
    if self._mode == Mode.TRAIN:
      log.info("Train step %d training loss: %f  - training perplexity: %f", step, loss, perplexity)
    for k, v in (additional_metrics or {}).items():
      self.metrics_logger.log(self.metrics_prefix, k, v, self._mode, step)

  def _buffer_metrics(self, metrics_buffer: Optional[MetricsBuffer], loss: Any, step: int,
                      additional_metrics: Optional[Mapping[str, Tuple[Any, Callable]]] = None) -> MetricsBuffer:
    if metrics_buffer is None:
      metrics_buffer = MetricsBuffer(step=step, losses=[loss])
    else:
      assert metrics_buffer.step == step
      if isinstance(metrics_buffer.losses[0], WeightedMetric) != isinstance(loss, WeightedMetric):
        raise TypeError("loss values must not mix weighted and scalar metrics")
      metrics_buffer.losses.append(loss)
    if additional_metrics is not None:
      for k, (v, op) in additional_metrics.items():
        if k not in metrics_buffer.additional_metrics:
          metrics_buffer.additional_metrics[k] = ([v], op)
        else:
          values = metrics_buffer.additional_metrics[k][0]
          if isinstance(values[0], WeightedMetric) != isinstance(v, WeightedMetric):
            raise TypeError(f"additional metric {k!r} must not mix weighted and scalar values")
          values.append(v)
    return metrics_buffer

  def _write_train_metrics(self):
    """Writes the metrics buffered for the previous optimizer step."""
    if self._prev_buffered_train_metrics is None:
      self._prev_buffered_train_metrics = self._buffered_train_metrics
      self._buffered_train_metrics = None
      return
    self._prev_buffered_train_metrics.step += 1   # train_steps is incremented after buffering
    self._write_metrics(self._prev_buffered_train_metrics)
    self._may_update_pbar(self._tqdm_train_metrics, step=self._prev_buffered_train_metrics.step,
                          loss=self._prev_buffered_train_metrics.loss)
    self._prev_buffered_train_metrics = self._buffered_train_metrics
    self._buffered_train_metrics = None

  def _write_metrics(self, metrics_buffer: MetricsBuffer):
    def to_np(v):
      if isinstance(v, torch.Tensor):
        return np.asarray(v.detach().float().cpu().numpy(), dtype=np.float32)
      if isinstance(v, list):
        return [to_np(x) for x in v]
      return v

    def apply_op(v, op):
      if isinstance(v, list) and v:
        weighted = [isinstance(x, WeightedMetric) for x in v]
        if any(weighted) and not all(weighted):
          raise TypeError("metrics must not mix weighted and scalar values")
        if all(weighted):
          if getattr(op, "__name__", "") in ("_weighted_metric_mean", "global_weighted_mean", "mean_of_means"):
            return op(v)
          v = [x.compute() for x in v]
      return op(to_np(v))

    self._log_metrics(loss=self._global_loss(metrics_buffer), step=metrics_buffer.step,
                      additional_metrics={k: apply_op(v, op) for k, (v, op) in
                                          metrics_buffer.additional_metrics.items()})
    self._check_kernel_status()

  def _check_kernel_status(self) -> None:
    """Raises when a kernel of the steps written so far reported an error (a bounded wait on a peer or a
    pipeline barrier that ran out, a bad argument, rows dropped by an expert-parallel receive buffer).
    Called where the loss has just been read back, so the check adds no synchronisation of its own; a
    step whose kernels failed is therefore reported at most one optimizer step late, before its
    parameters reach a checkpoint."""
    if self._device is not None and self._device.type == "cuda":
      from ..ops import _lib
      _lib.check_status(self._device)

  def _global_loss(self, metrics_buffer: MetricsBuffer) -> float:
    """Loss of the step over all data-parallel ranks (each rank buffered its own share)."""
    gs = self._grad_sync
    if gs is None or getattr(gs, "world", 1) == 1:
      return metrics_buffer.loss
    losses = metrics_buffer.losses
    if isinstance(losses[0], WeightedMetric):
      total = sum(_to_float(v.unreduced_sum) for v in losses)
      denom = sum(_to_float(v.denominator) for v in losses)
      total, denom = gs.reduce_scalars([total, denom])
      return _to_float(WeightedMetric(total, denom, losses[0].eps, losses[0].min_denom).compute())
    (mean,) = gs.reduce_scalars([metrics_buffer.loss])
    return mean / gs.world

  @contextlib.contextmanager
  def _switch_mode(self, mode: Mode):
    original = self._mode
    self._mode = mode
    try:
      yield
    finally:
      self._mode = original

  @property
  def _tqdm_train_metrics(self) -> List[str]:
    return ["loss", "perplexity", "learning_rate"]

  def _may_update_pbar(self, metrics: List[str], step: Optional[int] = None, loss: Any = None):
    if self._pbar is not None:
      self._pbar.update_metrics(metrics, self._mode, ndigits=3)
      self._pbar.update()
    if self.training_hooks and self._mode == Mode.TRAIN:
      self.training_hooks.on_train_step_end(self, step, loss)

  # ---- the loop ----------------------------------------------------------------------------
  def _is_update_step(self, train_example: Any) -> bool:
    ga = self.config.get_with_default("gradient_accumulation_steps", 1)
    val = None
    if isinstance(train_example, dict) and "is_update_step" in train_example:
      val = train_example["is_update_step"]
    elif hasattr(train_example, "is_update_step"):
      val = train_example.is_update_step
    if val is not None:
      return bool(np.asarray(val.cpu() if isinstance(val, torch.Tensor) else val).item())
    return self._iter_steps % ga == 0

  def train(self, train_ds: Iterable[Any], eval_ds: Optional[Iterable[Any]] = None, skip_jit: bool = False, *,
            cache_nnx_graph: bool = True) -> None:
    """Runs the training loop over `train_ds` (an iterable of batches)."""
    del skip_jit, cache_nnx_graph
    if eval_ds:
      self._run_eval(eval_ds)
    if self.config.max_steps is not None and self._pbar is None and self.config.pbar_description is not None:
      self._pbar = progress_bar.ProgressBar(metrics_prefix=self.metrics_prefix, metrics_logger=self.metrics_logger,
                                            initial_steps=self._train_steps, max_steps=self.config.max_steps,
                                            description=self.config.pbar_description)
    if self.training_hooks:
      self.training_hooks.on_train_start(self)

    train_iterator = iter(train_ds)
    index = 0
    t_start = time.perf_counter()
    while True:
      self._prof.maybe_activate(self._iter_steps)
      train_example = None
      if self.data_hooks:
        train_example = self.data_hooks.load_next_train_batch(self)
      else:
        try:
          train_example = next(train_iterator)
          if not self.is_managed_externally and index < self._iter_steps:
            index += 1     # resume: skip what was already trained on
            continue
          index += 1
        except StopIteration:
          pass
      if train_example is None:
        break
      if (not self.is_managed_externally and self.config.max_steps is not None
          and self._train_steps >= self.config.max_steps):
        break

      train_example = self._prepare_inputs(train_example)
      train_example = sharding_utils.shard_input(train_example, self.config.data_sharding_axis, self._device)

      self._throttler.wait_for_next()
      if self.training_hooks:
        self.training_hooks.on_train_step_start(self)

      metadata = self.custom_checkpoint_metadata()
      ga = self.config.get_with_default("gradient_accumulation_steps", 1)
      tags = {"step": metadata.get("global_step"), "role": metadata.get("role"),
              "micro_batch": self._iter_steps % ga, "mini_batch": self._train_steps}
      self._iter_steps += 1
      is_update = self._is_update_step(train_example)

      with self._perf_tracer.span("peft_train_step") as span, \
           self._perf_tracer_v2.span("peft_train_step", tags=tags) as span_v2:
        train_loss, aux, grad_norm = self._train_step(train_example, is_update)
        span.device_end([train_loss])
        span_v2.async_end([train_loss])

      self._throttler.add_computation(train_loss)
      buffered_loss = aux.primary_loss if isinstance(aux, LossOutput) else train_loss
      additional: Dict[str, Tuple[Any, Callable]] = {"grad_norm": (grad_norm, np.mean)}
      post_aux = aux
      if isinstance(aux, LossOutput):
        additional.update({name: (m, _metric_reducer(m)) for name, m in aux.aux_metrics.items()})
        post_aux = aux.aux_metrics
      self._buffered_train_metrics = self._buffer_metrics(self._buffered_train_metrics, loss=buffered_loss,
                                                          step=self._train_steps, additional_metrics=additional)
      self._post_process_train_step(post_aux)

      if is_update:
        self._train_steps += 1
        self._write_train_metrics()
        self.checkpoint_manager.save(self._train_steps, self.model, self.optimizer,
                                     save_only_lora_params=self._lora_enabled,
                                     custom_metadata=self.custom_checkpoint_metadata())
        if eval_ds and self._train_steps % self.config.eval_every_n_steps == 0:
          self._run_eval(eval_ds)
      self._prof.maybe_deactivate(self._iter_steps)

    self._throttler.wait_for_all()
    log.info("Train loop finished in: %.4f seconds", time.perf_counter() - t_start)
    if self.training_hooks:
      self.training_hooks.on_train_end(self)
    if not self.is_managed_externally:
      self.close()

  def _save_last_checkpoint(self):
    last = self.checkpoint_manager.latest_step()
    if last is None or last < self._train_steps:
      self.checkpoint_manager.save(self._train_steps, self.model, self.optimizer,
                                   save_only_lora_params=self._lora_enabled, force=True,
                                   custom_metadata=self.custom_checkpoint_metadata())

  @property
  def train_steps(self) -> int:
    return self._train_steps

  @property
  def iter_steps(self) -> int:
    return self._iter_steps

  def custom_checkpoint_metadata(self) -> Dict[str, Any]:
    return {}

  def close(self):
    """Flushes buffered metrics, forces the last checkpoint, closes logger and checkpointer."""
    self._write_train_metrics()
    if self._prev_buffered_train_metrics is not None:
      self._write_train_metrics()
    self._closing = True     # metadata providers may distinguish the final save from in-loop saves
    self._save_last_checkpoint()
    self.checkpoint_manager.close()
    self.metrics_logger.close()
    if self._pbar is not None:
      self._pbar.close()
      self._pbar = None

  def _run_eval(self, eval_ds: Iterable[Any]) -> None:
    log.info("Running evaluation on train step %d.", self._train_steps)
    eval_iterator = iter(eval_ds)
    with self._switch_mode(Mode.EVAL):
      eval_loss, eval_steps, weighted = 0.0, 0, False
      while True:
        if self.data_hooks:
          ex = self.data_hooks.load_next_eval_batch(self)
        else:
          ex = next(eval_iterator, None)
        if ex is None:
          break
        ex = self._prepare_inputs(ex)
        ex = sharding_utils.shard_input(ex, self.config.data_sharding_axis, self._device)
        if self.training_hooks:
          self.training_hooks.on_eval_step_start(self)
        loss, aux = self._eval_step(ex)
        buffered = aux.primary_loss if isinstance(aux, LossOutput) else loss
        additional = None
        post_aux = aux
        if isinstance(aux, LossOutput):
          weighted = True
          additional = {name: (m, _metric_reducer(m)) for name, m in aux.aux_metrics.items()}
          post_aux = aux.aux_metrics
        self._buffered_eval_metrics = self._buffer_metrics(self._buffered_eval_metrics, loss=buffered,
                                                           step=self._train_steps, additional_metrics=additional)
        self._post_process_eval_step(post_aux)
        eval_loss += _to_float(loss)
        eval_steps += 1
      if eval_steps == 0:
        log.warning("No eval examples found. Skipping eval metrics logging.")
        return
      buf = self._buffered_eval_metrics
      if weighted:
        eval_loss = buf.loss
      self._write_metrics(buf)
      log.info("Train step %d eval loss: %f - eval perplexity: %f", self._train_steps,
               self.metrics_logger.get_metric(self.metrics_prefix, "loss", "eval"),
               self.metrics_logger.get_metric(self.metrics_prefix, "perplexity", "eval"))
      self._buffered_eval_metrics = None
      if self.training_hooks:
        self.training_hooks.on_eval_step_end(self, eval_loss)


def _default_gen_model_input_fn(x: Any) -> Dict[str, Any]:
  """TrainingInput / dict -> kwargs of the default loss."""
  if isinstance(x, TrainingInput):
    d = {"input_tokens": x.input_tokens, "input_mask": x.input_mask}
    if x.images is not None:
      d["images"] = x.images
    return d
  if isinstance(x, dict):
    return x
  return dict(x)


def _default_loss_fn(model: torch.nn.Module, input_tokens: torch.Tensor, input_mask: torch.Tensor,
                     positions: Optional[torch.Tensor] = None, attention_mask: Optional[torch.Tensor] = None,
                     images: Any = None, segment_ids: Optional[torch.Tensor] = None) -> LossOutput:
  """Next-token negative log-likelihood: logits[:, :-1] against tokens[:, 1:], masked by
  input_mask[:, 1:], as an unreduced sum with denominator sum(mask) and eps 1e-8
  (tunix/sft/peft_trainer.py:1230-1263).

  `attention_mask=None` means causal attention (right-padded or unpadded rows). When the model
  exposes `head_weight()` the lm_head and the log-softmax run fused and sequence-chunked, so
  the `[B, L, V]` logits are never materialised.
  """
  from ..ops import functional as F
  kwargs = {} if images is None else {"images": images}
  if segment_ids is not None:
    kwargs["segment_ids"] = segment_ids
  target_tokens = input_tokens[:, 1:]
  target_mask = input_mask[:, 1:].to(torch.float32)
  if hasattr(model, "head_weight"):
    hidden, _ = model(input_tokens, positions, None, attention_mask, skip_lm_head=True, **kwargs)
    # score every position against the next token; the last position has no target and is
    # masked out, which avoids copying hidden[:, :-1]
    shifted = torch.roll(input_tokens, shifts=-1, dims=1)
    mask_full = torch.cat([target_mask, target_mask.new_zeros(target_mask.shape[0], 1)], dim=1)
    cap = getattr(model.config, "final_logit_softcap", None) or 0.0
    logp, _ = F.linear_logprob(hidden, model.head_weight(), shifted, softcap=cap)
    unreduced = -(logp * mask_full).sum()
    return LossOutput(primary_loss=WeightedMetric(unreduced, target_mask.sum(), eps=1e-8), aux_metrics={})
  else:
    logits, _ = model(input_tokens, positions, None, attention_mask, **kwargs)
    logp, _ = F.ref.selective_log_softmax(logits[:, :-1], target_tokens)
  unreduced = -(logp * target_mask).sum()
  return LossOutput(primary_loss=WeightedMetric(unreduced, target_mask.sum(), eps=1e-8), aux_metrics={})
