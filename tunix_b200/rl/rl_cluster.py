"""RL cluster: owns the models of every role and the engines built on them.

Roles (actor, critic, reference, reward, rollout) map to meshes over ranks
(`ClusterConfig.role_to_mesh`). The cluster places each model on its role's ranks, shares
storage where the reference does (actor and rollout on the same mesh share one model; with LoRA
the reference shares the actor's frozen backbone), builds the rollout engine, the inference
worker (critic / reference / reward) and the actor / critic trainers, buffers RL metrics per
global step, and synchronises trainer weights into the rollout engine
(tunix/rl/rl_cluster.py:73-1252).
"""
from __future__ import annotations

import contextlib
import copy
import dataclasses
import gc
import itertools
import logging
from typing import Any, Callable, Dict, List, Mapping, Optional, Tuple, Union

import numpy as np
import torch

from ..common.configs import ClusterConfig, RolloutConfig
from ..common.datatypes import Mode, Role
from ..generate import tokenizer_adapter
from ..perf import trace as perf_trace
from ..sft import metrics_logger as ml
from ..sft import sharding_utils
from ..sft import utils as sft_utils
from . import common, reshard
from . import trainer as rl_trainer
from . import utils as rl_utils
from .inference import inference_worker as iw
from .rollout import base_rollout, vanilla_rollout

log = logging.getLogger(__name__)
MetricsT = Dict[str, Tuple[Any, Optional[Callable]]]


@dataclasses.dataclass
class MetricsBuffer:
  global_steps: int
  metrics: Dict[str, Tuple[List[Any], Optional[Callable]]] = dataclasses.field(default_factory=dict)
  mode: str = "train"


def _device_of(model: torch.nn.Module):
  try:
    return next(model.parameters()).device
  except StopIteration:
    return None


class RLEngine:
  """See the module docstring. `RLCluster` is an alias."""

  def __init__(self, *, actor: torch.nn.Module, critic: Optional[torch.nn.Module] = None,
               reference: Optional[torch.nn.Module] = None, reward: Optional[torch.nn.Module] = None,
               tokenizer: Any, cluster_config: ClusterConfig, perf_config: Any = None):
    self.cluster_config = cluster_config
    self.perf_config = perf_config
    self.r2m = cluster_config.role_to_mesh
    self._anchor_policy_state: Optional[Dict[str, torch.Tensor]] = None
    # `sync_weights` also copies the start-of-step weights to pinned host memory for learners that score with the
    # old policy (`get_actor_per_token_logps`); a learner that never does may switch the copy off
    self.snapshot_anchor_on_sync = True
    if cluster_config.rollout_config is None:
      raise ValueError("`cluster_config.rollout_config` cannot be None.")
    if isinstance(cluster_config.rollout_config, dict) and not cluster_config.rollout_config.get(Mode.TRAIN):
      raise ValueError("Rollout config is a dict but missing a train config. Provided config: "
                       f"{cluster_config.rollout_config}")
    self._backbone_sharing_map = self._init_backbone_sharing_map(actor, reference)
    self.train_actor = self._load_model(actor, self.r2m.get(Role.ACTOR))
    if Role.ROLLOUT in self._backbone_sharing_map[Role.ACTOR]:
      self.rollout_actor = self.train_actor
    elif cluster_config.rollout_engine == "vanilla" or isinstance(cluster_config.rollout_engine, type):
      dt = self.get_rollout_config(Mode.TRAIN).data_type
      self.rollout_actor = self._load_model(copy.deepcopy(actor), self.r2m.get(Role.ROLLOUT), dt)
    else:
      self.rollout_actor = self.train_actor
    self.reference = self._load_model(reference, self.r2m.get(Role.REFERENCE)) if reference is not None else None
    if self.reference is not None and Role.REFERENCE in self._backbone_sharing_map[Role.ACTOR]:
      if not rl_utils.is_sharing_backbone(self.reference, self.train_actor):
        log.warning("Reference model and actor model are colocated but do not share the same backbone. This "
                    "will result in an unnecessary model copy and increased HBM usage.")
    self.critic = self._load_model(critic, self.r2m.get(Role.CRITIC)) if critic is not None else None
    self.reward = self._load_model(reward, self.r2m.get(Role.REWARD)) if reward is not None else None
    self.tokenizer = tokenizer_adapter.TokenizerAdapter(tokenizer) if tokenizer is not None and not isinstance(
        tokenizer, tokenizer_adapter.TokenizerAdapter) else tokenizer
    self._rl_metrics_logger = ml.MetricsLogger(cluster_config.training_config.metrics_logging_options)
    self._buffered_train_metrics: List[MetricsBuffer] = []
    self._buffered_eval_metrics: List[MetricsBuffer] = []
    self._external_metrics_logger = None
    self._init_engine()
    gc.collect()
    self.global_steps = 0

  # ---- construction ---------------------------------------------------------------------
  def _init_backbone_sharing_map(self, actor, reference) -> Dict[Role, List[Role]]:
    """Which roles may alias the actor's storage: the rollout when it runs on the actor's mesh,
    the reference when the actor trains LoRA adapters on the same mesh."""
    m: Dict[Role, List[Role]] = {Role.ACTOR: []}
    am = self.r2m.get(Role.ACTOR)
    if self.r2m.get(Role.ROLLOUT) == am and self.cluster_config.rollout_engine == "vanilla":
      m[Role.ACTOR].append(Role.ROLLOUT)
    if reference is not None and self.r2m.get(Role.REFERENCE) == am and sft_utils.is_lora_enabled(actor):
      m[Role.ACTOR].append(Role.REFERENCE)
    return m

  def _load_model(self, model: torch.nn.Module, mesh: Any, data_type: Optional[torch.dtype] = None):
    if model is None:
      return None
    model = reshard.reshard_model_to_mesh(model, mesh)
    if data_type is not None and next(model.parameters()).dtype != data_type:
      model.to(data_type)
    return model

  def _shard_actor(self):
    """An actor mesh of several ranks trains data-parallel with sharded optimizer state: parameters move into a
    flat store whose bf16 replica stays resident on every rank. A rollout engine that shares the module reads each
    update in place (`sync_weights` has nothing to copy); a tensor-parallel rollout re-shards from the store."""
    actor_mesh = self.r2m.get(Role.ACTOR)
    if actor_mesh is None or getattr(actor_mesh, "size", 1) <= 1 or not getattr(actor_mesh, "contains_me", True):
      return None
    import torch.distributed as torch_dist
    if not (torch_dist.is_available() and torch_dist.is_initialized()):
      return None
    from ..dist import fsdp
    axis = "fsdp" if "fsdp" in actor_mesh.axis_names else actor_mesh.axis_names[0]
    if not hasattr(self.train_actor, "flat_store"):
      fsdp.shard_model(self.train_actor, actor_mesh, axis)
    return fsdp.GradSync(self.train_actor, actor_mesh, axis)

  def _init_engine(self):
    cfg = self.cluster_config
    rc = self.get_rollout_config(Mode.TRAIN)
    actor_sync = self._shard_actor()          # before the rollout engine: it may slice the flat store
    mcfg = getattr(self.rollout_actor, "config", None)
    engine = cfg.rollout_engine
    if isinstance(engine, type) and issubclass(engine, base_rollout.BaseRollout):
      self._rollout = engine(rollout_actor=self.rollout_actor, tokenizer=self.tokenizer,
                             mesh=self.r2m.get(Role.ROLLOUT), rollout_config=rc)
    elif engine == "vanilla":
      if mcfg is None:
        raise ValueError("the vanilla rollout engine needs a model with a `config` (layers, kv heads, head dim)")
      cache = base_rollout.CacheConfig(cache_size=rc.kv_cache_size, num_layers=mcfg.num_layers,
                                       num_kv_heads=mcfg.num_kv_heads, head_dim=mcfg.head_dim)
      self._rollout = vanilla_rollout.VanillaRollout(self.rollout_actor, self.tokenizer, cache)
    elif engine == "native":
      from .rollout import native_rollout
      self._rollout = native_rollout.NativeRollout(self.rollout_actor, self.tokenizer, rc,
                                                   mesh=self.r2m.get(Role.ROLLOUT))
    elif engine == "vllm":
      from .rollout import vllm_rollout
      self._rollout = vllm_rollout.VllmRollout(self.rollout_actor, self.tokenizer, rc,
                                               mesh=self.r2m.get(Role.ROLLOUT))
    elif engine == "sglang_jax":
      from .rollout import sglang_jax_rollout
      self._rollout = sglang_jax_rollout.SglangJaxRollout(self.rollout_actor, self.tokenizer, rc,
                                                          mesh=self.r2m.get(Role.ROLLOUT))
    else:
      raise NotImplementedError(f"Rollout engine {engine} not supported")
    models = {}
    if self.critic is not None:
      models["critic"] = self.critic
    if self.reference is not None:
      models["reference"] = self.reference
    if self.reward is not None:
      models["reward"] = self.reward
    self._inference_worker = iw.InferenceWorker(models)

    tc = cfg.training_config
    if self.perf_config is not None:
      from ..perf import export as perf_export
      export_fn = getattr(self.perf_config, "custom_export_fn", None) or \
          perf_export.PerfMetricsExport.from_cluster_config(cfg)
      devices = sorted({r for m in self.r2m.values() if m is not None for r in m.ranks()})
      self._perf = perf_trace.PerfTracer(devices, export_fn)
    else:
      self._perf = perf_trace.NoopTracer()
    self._perf_v2 = perf_trace.NoopTracer()
    root = tc.checkpoint_root_directory
    actor_cfg = copy.copy(tc)
    if root:
      actor_cfg.checkpoint_root_directory = f"{root}/actor"
    self._actor_trainer = rl_trainer.Trainer(
        model=self.train_actor, optimizer=tc.actor_optimizer, training_config=_as_training_config(actor_cfg),
        custom_checkpoint_metadata_fn=lambda: {
            "global_step": self.global_steps + (0 if self._actor_trainer._closing else 1), "role": "actor"},
        metrics_logger=self._rl_metrics_logger, perf_tracer=self._perf, perf_tracer_v2=self._perf_v2)
    if actor_sync is not None:
      self._actor_trainer.with_grad_sync(actor_sync)
    del self.train_actor
    self._maybe_offload_model_to_cpu(self._actor_trainer.model, Role.ACTOR)
    if self.critic is not None:
      critic_cfg = copy.copy(tc)
      if root:
        critic_cfg.checkpoint_root_directory = f"{root}/critic"
      self._critic_trainer = rl_trainer.Trainer(
          model=self.critic, optimizer=tc.critic_optimizer or tc.actor_optimizer,
          training_config=_as_training_config(critic_cfg),
          custom_checkpoint_metadata_fn=lambda: {
              "global_step": self.global_steps + (0 if self._critic_trainer._closing else 1), "role": "critic"},
          metrics_logger=self._rl_metrics_logger, perf_tracer=self._perf, perf_tracer_v2=self._perf_v2)
      del self.critic
    # anchor snapshot of the start-of-step actor weights (host-pinned when the actor is on a GPU)
    if _device_of(self._actor_trainer.model) is not None and _device_of(self._actor_trainer.model).type == "cuda":
      self._anchor_policy_state = None

  # ---- memory placement --------------------------------------------------------------------
  def _maybe_load_model_from_cpu(self, model, role: Role):
    if self.cluster_config.offload_to_cpu and model is not None:
      rl_utils.put_params_on_memory_kind(model, "device")

  def _maybe_offload_model_to_cpu(self, model, role: Role):
    if self.cluster_config.offload_to_cpu and model is not None:
      rl_utils.put_params_on_memory_kind(model, "pinned_host")

  # ---- accessors -------------------------------------------------------------------------------
  @property
  def rollout(self) -> base_rollout.BaseRollout:
    return self._rollout

  @property
  def inference_worker(self) -> iw.InferenceWorker:
    return self._inference_worker

  @property
  def actor_trainer(self) -> rl_trainer.Trainer:
    return self._actor_trainer

  @property
  def critic_trainer(self) -> rl_trainer.Trainer:
    return self._critic_trainer

  @property
  def perf(self):
    return self._perf

  @property
  def perf_v2(self):
    return self._perf_v2

  def close(self):
    for m in self._buffered_train_metrics + self._buffered_eval_metrics:
      self._log_metrics(m)
    self._buffered_train_metrics, self._buffered_eval_metrics = [], []
    self.actor_trainer.close()
    if hasattr(self, "_critic_trainer"):
      self._critic_trainer.close()

  # ---- metrics -------------------------------------------------------------------------------------
  def _log_metrics(self, metrics_buffer: MetricsBuffer) -> None:
    for name, (value, op) in metrics_buffer.metrics.items():
      try:
        vals = [v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else v for v in value]
        agg = np.array(vals)
      except Exception:
        log.warning("Skipping metric %s: Could not convert to numpy array.", name)
        continue
      if agg.dtype.kind in {"U", "S"} or (agg.dtype.kind == "O" and agg.size > 0 and
                                          isinstance(agg.ravel()[0], (str, np.str_))):
        log.info("Rollout string metric %s: %s", name, agg)
        continue
      if agg.dtype.kind == "O":
        try:
          agg = np.concatenate([np.atleast_1d(np.asarray(v, dtype=np.float64)) for v in vals])
        except Exception:
          continue
      if op is not None and agg.size > 0:
        agg = op(agg)
      prefix, short = name.split("/", 1) if "/" in name else ("global", name)
      self._rl_metrics_logger.log(prefix, short, agg, metrics_buffer.mode, metrics_buffer.global_steps)
    if self._external_metrics_logger is not None:
      self._external_metrics_logger(metrics_buffer)

  def with_external_metrics_logger(self, external_metrics_logger: Callable[[MetricsBuffer], None]):
    self._external_metrics_logger = external_metrics_logger
    return self

  # RL metrics are kept in a ledger keyed by (mode, global step) and written once the run has moved past
  # their step, so everything that belongs to one step - rollout statistics recorded by the producer thread,
  # rewards, trainer-side values - lands in one logger call, in step order.
  def _ledger(self, mode: Mode) -> List[MetricsBuffer]:
    return self._buffered_train_metrics if mode == Mode.TRAIN else self._buffered_eval_metrics

  def _record(self, metrics: MetricsT, mode: Mode, step: int) -> None:
    ledger = self._ledger(mode)
    page = next((m for m in reversed(ledger) if m.global_steps == step), None)
    if page is None:
      page = MetricsBuffer(step, mode=str(mode))
      ledger.append(page)
      ledger.sort(key=lambda m: m.global_steps)
    for name, (value, op) in metrics.items():
      page.metrics.setdefault(name, ([], op))[0].append(value)

  def _write_finished_steps(self) -> None:
    for ledger in (self._buffered_train_metrics, self._buffered_eval_metrics):
      while ledger and ledger[0].global_steps < self.global_steps:
        self._log_metrics(ledger.pop(0))

  def buffer_metrics(self, metrics: MetricsT, mode: Mode = Mode.TRAIN) -> None:
    """Records metrics of the current global step; steps the run has left behind are written out."""
    self._write_finished_steps()
    self._record(metrics, mode, self.global_steps)

  def buffer_metrics_async(self, metrics: MetricsT, mode: Mode = Mode.TRAIN, step: int = 0) -> None:
    """Like `buffer_metrics` for a producer that runs ahead of (or behind) the trainer: the caller names the
    step the values belong to."""
    self._record(metrics, mode, step)
    self._write_finished_steps()

  # ---- training ----------------------------------------------------------------------------------------
  def train(self, role: Role, train_ds: Any, eval_ds: Any, skip_jit: bool = False) -> None:
    if role == Role.ACTOR:
      self.update_actor(train_ds, eval_ds, skip_jit)
    elif role == Role.CRITIC:
      self.update_critic(train_ds, eval_ds, skip_jit)
    else:
      raise ValueError(f"Unsupported role for train: {role}")

  def update_actor(self, train_ds, eval_ds, skip_jit=False):
    self._maybe_load_model_from_cpu(self.actor_trainer.model, Role.ACTOR)
    self._anchor_ready()       # the snapshot of the old weights is complete before they change
    with self._perf.span_group("actor_training"):
      self.actor_trainer.train(train_ds, eval_ds, skip_jit)
    self._maybe_offload_model_to_cpu(self.actor_trainer.model, Role.ACTOR)

  def eval_actor(self, eval_ds: Any) -> Any:
    if eval_ds is None:
      return None
    self._maybe_load_model_from_cpu(self.actor_trainer.model, Role.ACTOR)
    res = self.actor_trainer._run_eval(eval_ds)
    self._maybe_offload_model_to_cpu(self.actor_trainer.model, Role.ACTOR)
    return res

  def update_critic(self, train_ds, eval_ds, skip_jit=False):
    self._maybe_load_model_from_cpu(self.critic_trainer.model, Role.CRITIC)
    with self._perf.span_group("critic_training"):
      self._critic_trainer.train(train_ds, eval_ds, skip_jit)
    self._maybe_offload_model_to_cpu(self.critic_trainer.model, Role.CRITIC)

  # ---- inference -------------------------------------------------------------------------------------------
  def get_rollout_config(self, mode: Mode) -> RolloutConfig:
    rc = self.cluster_config.rollout_config
    return rc[mode] if isinstance(rc, dict) else rc

  def _render_prompts(self, prompts, apply_chat_template: bool) -> List[str]:
    if not apply_chat_template:
      return list(prompts)
    if self.tokenizer is None:
      raise ValueError("Tokenizer must be initialized to use chat templates.")
    return [self.tokenizer.apply_chat_template(chat, add_generation_prompt=True, tokenize=False, enable_thinking=False)
            for chat in prompts]

  @staticmethod
  def _join_rollouts(parts: List[base_rollout.RolloutOutput]) -> base_rollout.RolloutOutput:
    """One `RolloutOutput` from the outputs of consecutive micro-batches (optional fields stay optional)."""
    def flat(field: str, present: bool):
      return [x for part in parts for x in getattr(part, field)] if present else None
    head = parts[0]
    return base_rollout.RolloutOutput(
        text=flat("text", True), tokens=flat("tokens", True),
        logits=flat("logits", head.logits is not None and len(head.logits) > 0),
        logprobs=flat("logprobs", head.logprobs is not None),
        left_padded_prompt_tokens=np.concatenate([part.left_padded_prompt_tokens for part in parts], axis=0))

  def generate(self, prompts, apply_chat_template: bool = False, mode: Mode = Mode.TRAIN,
               micro_batch_size: Optional[int] = None, trace_tags: Optional[Mapping[str, Any]] = None,
               max_generation_steps: Optional[int] = None) -> base_rollout.RolloutOutput:
    """Completions for `prompts` (strings, or chats when `apply_chat_template`) from the rollout engine, generated
    `micro_batch_size` prompts at a time under the rollout configuration of `mode`."""
    texts = self._render_prompts(prompts, apply_chat_template)
    if not texts:
      raise ValueError("Cannot generate from an empty list of prompts.")
    rc = self.get_rollout_config(mode)
    if max_generation_steps is not None:
      rc = dataclasses.replace(rc, max_tokens_to_generate=max_generation_steps)
    engine_model = self.rollout.model()
    self._maybe_load_model_from_cpu(engine_model, Role.ROLLOUT)
    try:
      with self._perf.span("rollout") as span, \
           self._perf_v2.span("rollout", tags={"role": Role.ROLLOUT.value, **(trace_tags or {})}) as span_v2:
        parts = [self.rollout.generate(texts[sl], rc)
                 for sl in rl_utils.chunk_slices_by_size(len(texts), micro_batch_size or len(texts))]
        produced = [part.tokens for part in parts]
        span.device_end(produced)
        span_v2.async_end(produced)
    finally:
      self._maybe_offload_model_to_cpu(engine_model, Role.ROLLOUT)
    return self._join_rollouts(parts)

  def per_token_logps(self, role: Role, prompt_tokens, completion_tokens, pad_id: int, eos_id: int,
                      micro_batch_size: Optional[int] = None, segment_ids=None, **kwargs):
    if role == Role.REFERENCE:
      return self.get_ref_per_token_logps(prompt_tokens, completion_tokens, pad_id, eos_id, micro_batch_size,
                                          segment_ids, **kwargs)
    if role == Role.ACTOR:
      return self.get_actor_per_token_logps(prompt_tokens, completion_tokens, pad_id, eos_id, micro_batch_size,
                                            segment_ids=segment_ids, **kwargs)
    raise ValueError(f"Unsupported role for per_token_logps: {role}")

  def _place(self, x, model):
    if x is None:
      return None
    if isinstance(x, np.ndarray):
      x = torch.from_numpy(x)
    dev = _device_of(model)
    return x.to(dev) if dev is not None else x

  def get_ref_per_token_logps(self, prompt_tokens, completion_tokens, pad_id: int, eos_id: int,
                              micro_batch_size: Optional[int] = None, segment_ids=None, segment_positions=None):
    B = prompt_tokens.shape[0]
    if B == 0:
      raise ValueError("Cannot get reference log probabilities from an empty batch.")
    mb = micro_batch_size or B
    ref = self.inference_worker.get_model("reference")
    self._maybe_load_model_from_cpu(ref, Role.REFERENCE)
    p, c = self._place(prompt_tokens, ref), self._place(completion_tokens, ref)
    s, sp = self._place(segment_ids, ref), self._place(segment_positions, ref)
    temperature = self.get_rollout_config(Mode.TRAIN).temperature
    outs = []
    # with a LoRA actor sharing the backbone, the reference is the actor with adapters disabled
    with _adapters_disabled(ref if self._ref_is_actor_backbone(ref) else None):
      for sl in rl_utils.chunk_slices_by_size(B, mb):
        outs.append(self.inference_worker.get_ref_per_token_logps(
            p[sl], c[sl], pad_id, eos_id, temperature=temperature,
            segment_ids=None if s is None else s[sl], segment_positions=None if sp is None else sp[sl]))
    self._maybe_offload_model_to_cpu(ref, Role.REFERENCE)
    return torch.cat(outs, dim=0)

  def _ref_is_actor_backbone(self, ref) -> bool:
    return ref is self.actor_trainer.model

  def get_old_per_token_logps(self, prompt_tokens, completion_tokens, micro_batch_size: Optional[int] = None):
    B = prompt_tokens.shape[0]
    if B == 0:
      raise ValueError("Cannot get old log probabilities from an empty batch.")
    mb = micro_batch_size or B
    model = self.rollout.model()
    self._maybe_load_model_from_cpu(model, Role.ROLLOUT)
    p, c = self._place(prompt_tokens, model), self._place(completion_tokens, model)
    outs = [self.rollout.get_per_token_logps(p[sl], c[sl]) for sl in rl_utils.chunk_slices_by_size(B, mb)]
    self._maybe_offload_model_to_cpu(model, Role.ROLLOUT)
    return torch.cat(outs, dim=0)

  def get_actor_per_token_logps(self, prompt_tokens, completion_tokens, pad_id: int, eos_id: int,
                                micro_batch_size: Optional[int] = None, temperature: Optional[float] = None,
                                segment_ids=None, segment_positions=None):
    """Log-probabilities under the start-of-step actor (the anchor snapshot taken by the last
    `sync_weights`), scaled by the rollout temperature so they are comparable to the sampler's."""
    if temperature is None:
      temperature = self.get_rollout_config(Mode.TRAIN).temperature
    B = prompt_tokens.shape[0]
    if B == 0:
      raise ValueError("Cannot get actor log probabilities from an empty batch.")
    if self._anchor_policy_state is None:
      raise ValueError("Anchor policy state is not initialized. Please run `sync_weights` first.")
    mb = micro_batch_size or B
    model = self.actor_trainer.model
    p, c = self._place(prompt_tokens, model), self._place(completion_tokens, model)
    s, sp = self._place(segment_ids, model), self._place(segment_positions, model)
    outs = []
    self._anchor_ready(host=True)
    with _swapped_params(model, self._anchor_policy_state):
      for sl in rl_utils.chunk_slices_by_size(B, mb):
        outs.append(common.compute_per_token_logps(
            model, p[sl], c[sl], pad_id, eos_id, stop_gradient=True, temperature=temperature,
            segment_ids=None if s is None else s[sl], segment_positions=None if sp is None else sp[sl]))
    return torch.cat(outs, dim=0)

  @torch.no_grad()
  def sync_weights(self):
    """Pushes the actor's (LoRA-only when LoRA is enabled) parameters into the rollout engine and
    refreshes the host-pinned anchor snapshot; advances the global step."""
    model = self.actor_trainer.model
    lora = sft_utils.is_lora_enabled(model)
    params = {n: p for n, p in model.named_parameters() if (getattr(p, "is_lora", False) or not lora)}
    self.rollout.update_params(params, ("lora",) if lora else None)
    if self.snapshot_anchor_on_sync:
      self._snapshot_anchor(params)
    gc.collect()
    self.global_steps += 1

  def weight_sync_ms(self) -> Optional[float]:
    """Device time of the last trainer -> rollout transfer, when the rollout engine measures it."""
    fn = getattr(self.rollout, "weight_sync_ms", None)
    return fn() if fn is not None else None

  def _snapshot_anchor(self, params: Mapping[str, torch.Tensor]) -> None:
    """Copies the start-of-step weights to pinned host buffers that are allocated once and reused.

    On a GPU the copy runs on a side stream so the rollout that follows overlaps it; whoever changes
    the weights next (`train`) or reads the snapshot first waits for it through `_anchor_ready`."""
    bufs = self._anchor_policy_state or {}
    cuda = any(p.is_cuda for p in params.values())
    if not cuda:
      self._anchor_policy_state = {n: p.detach().clone() for n, p in params.items()}
      self._anchor_event = None
      return
    if getattr(self, "_anchor_stream", None) is None:
      self._anchor_stream = torch.cuda.Stream()
    main = torch.cuda.current_stream()
    side = self._anchor_stream
    side.wait_stream(main)
    out = {}
    with torch.cuda.stream(side):
      for n, p in params.items():
        t = bufs.get(n)
        if t is None or t.shape != p.shape or t.dtype != p.dtype:
          t = torch.empty(p.shape, dtype=p.dtype, device="cpu", pin_memory=True)
        t.copy_(p.detach(), non_blocking=True)
        out[n] = t
      ev = torch.cuda.Event()
      ev.record(side)
    self._anchor_policy_state = out
    self._anchor_event = ev

  def _anchor_ready(self, host: bool = False) -> None:
    ev = getattr(self, "_anchor_event", None)
    if ev is None:
      return
    if host:
      ev.synchronize()
    else:
      torch.cuda.current_stream().wait_event(ev)

  def get_values(self, prompt_tokens, completion_tokens, pad_id: int, eos_id: int):
    m = self.inference_worker.get_model("critic")
    return self.inference_worker.get_values(self._place(prompt_tokens, m), self._place(completion_tokens, m),
                                            pad_id, eos_id)

  def get_rewards(self, prompt_tokens, completion_tokens, pad_id: int, eos_id: int):
    m = self.inference_worker.get_model("reward")
    return self.inference_worker.get_rewards(self._place(prompt_tokens, m), self._place(completion_tokens, m),
                                             pad_id, eos_id)


@contextlib.contextmanager
def _adapters_disabled(model):
  """Temporarily zeroes the LoRA scale of every adapter (reference = frozen backbone)."""
  if model is None:
    yield
    return
  saved = []
  for mod in model.modules():
    sc = getattr(mod, "lora_scale", None)
    if isinstance(sc, dict) and sc:
      saved.append((mod, dict(sc)))
      for k in sc:
        sc[k] = 0.0
  try:
    yield
  finally:
    for mod, sc in saved:
      mod.lora_scale.update(sc)


@contextlib.contextmanager
def _swapped_params(model: torch.nn.Module, state: Mapping[str, torch.Tensor]):
  """Runs the body with `state` loaded into the model's parameters, then restores them."""
  cur = dict(model.named_parameters())
  saved = {}
  with torch.no_grad():
    for n, t in state.items():
      p = cur[n]
      saved[n] = p.detach().clone()
      p.copy_(t.to(p.device, p.dtype))
  try:
    yield
  finally:
    with torch.no_grad():
      for n, t in saved.items():
        cur[n].copy_(t)


def _as_training_config(cfg):
  return cfg


RLCluster = RLEngine
