"""Base class of the RL learners: the global-step / mini-batch / micro-batch loops with a
producer thread that generates rollouts and computes advantages while the trainer consumes
them (tunix/rl/rl_learner.py:54-834).

Batch hierarchy: a dataloader batch (x G samples) is one *global step*; it is cut into
*mini-batches* (one optimizer update each), which are cut into *micro-batches* (one
forward/backward each). Rollout and log-prob micro-batch sizes may differ from the training
one; the producer merges micro-batches up to their least common multiple before it calls
`_generate_and_compute_advantage`, then splits the result back.
"""
from __future__ import annotations

import abc
import itertools
import logging
import math
from concurrent import futures
from typing import Any, Dict, Iterable, Iterator, List, Optional, Sequence

import numpy as np
import torch

from ..common.datatypes import Mode, Role
from ..sft import utils as sft_utils
from . import common, function_registry
from . import rl_cluster as rl_engine_lib
from . import utils as rl_utils
from .queue import data_queue as queue_lib

log = logging.getLogger(__name__)
TrainingInputT = Dict[str, Any]


def _repeat_tree(example: TrainingInputT, n: int) -> TrainingInputT:
  out = {}
  for k, v in example.items():
    if isinstance(v, torch.Tensor):
      out[k] = v.repeat_interleave(n, dim=0)
    elif isinstance(v, np.ndarray):
      out[k] = np.repeat(v, n, axis=0)
    elif isinstance(v, (list, tuple)):
      out[k] = [x for x in v for _ in range(n)]
    else:
      out[k] = v
  return out



def sft_utils_device(model) -> Optional[torch.device]:
  try:
    return next(model.parameters()).device
  except StopIteration:
    return None


def _bind_producer_thread(device) -> None:
  """The rollout producer thread launches kernels: it must use the trainer's GPU, not device 0."""
  if device is not None and device.type == "cuda":
    torch.cuda.set_device(device)


class RLLearner(abc.ABC):

  def __init__(self, rl_engine: Optional[rl_engine_lib.RLEngine] = None, algo_config: Any = None,
               reward_fns: Any = None, metric_fns: Optional[Sequence[Any]] = None,
               data_shuffle_seed: Optional[int] = None, rl_cluster: Optional[rl_engine_lib.RLEngine] = None):
    rl_engine = rl_engine if rl_engine is not None else rl_cluster
    self.rl_engine = rl_engine
    self.algo_config = algo_config
    self.reward_manager = function_registry.get_reward_manager(algo_config.reward_manager)(
        reward_fns=reward_fns, algo_config=algo_config)
    self.metric_fns = metric_fns or []
    self.rl_engine.actor_trainer.is_managed_externally = True
    if hasattr(self.rl_engine, "_critic_trainer"):
      self.rl_engine.critic_trainer.is_managed_externally = True
    self._data_shuffle_rng = (np.random.default_rng(data_shuffle_seed) if data_shuffle_seed is not None else None)
    self._training_config = self.rl_engine.cluster_config.training_config
    if self._training_config.max_seq_token_per_tpu is not None:
      rc = self.rl_engine.get_rollout_config(Mode.TRAIN)
      rl_utils.validate_packing_budget(
          self._training_config.max_seq_token_per_tpu, getattr(rc, "max_prompt_length", 1000000),
          getattr(algo_config, "max_response_length", None) or rc.max_tokens_to_generate)
    self.rl_engine.global_steps = self.rl_engine.actor_trainer.restored_global_step()
    self._iter_steps = 0
    self._eval_iter_steps = 0
    # an engine with its own copy of the weights (vLLM) needs the transfer even when `model()` is the actor
    self.should_sync_weights = getattr(self.rl_engine.rollout, "holds_own_weights", False) or \
        not rl_utils.is_sharing_weights(self.rl_engine.actor_trainer.model, self.rl_engine.rollout.model())
    r2m = self.rl_engine.cluster_config.role_to_mesh
    self.can_enable_async_rollout = r2m.get(Role.ACTOR) != r2m.get(Role.ROLLOUT)
    self.executor = futures.ThreadPoolExecutor(max_workers=1, initializer=_bind_producer_thread,
                                               initargs=(sft_utils_device(self.rl_engine.actor_trainer.model),))
    self._last_iter_step = self.rl_engine.actor_trainer.iter_steps
    self._rollout_micro_batch_size = self._training_config.rollout_micro_batch_size
    self._compute_logps_micro_batch_size = self._training_config.compute_logps_micro_batch_size
    sft_utils.show_hbm_usage(title="RLLearner init")

  # ---- to implement ----------------------------------------------------------------------
  @abc.abstractmethod
  def _generate_and_compute_advantage(self, training_input: TrainingInputT, mode: Mode = Mode.TRAIN):
    ...

  @abc.abstractmethod
  def _compute_trajectory_ids(self, example: TrainingInputT, steps: int) -> List[str]:
    ...

  @abc.abstractmethod
  def _num_iterations(self) -> int:
    ...

  @abc.abstractmethod
  def _num_generations(self) -> int:
    ...

  # ---- helpers ------------------------------------------------------------------------------
  def _compute_rewards(self, prompts: List[str], completions: List[str], mode: Mode, step: Optional[int] = None,
                       **kwargs) -> np.ndarray:
    """Sum of all reward functions per (prompt, completion); per-function values are logged."""
    if "mode" in kwargs:
      raise ValueError(f"kwargs already contains mode as a key: {kwargs}")
    kwargs["mode"] = str(mode)
    info = self.reward_manager(prompts=prompts, completions=completions, **kwargs)
    if step is not None:
      self.rl_engine.buffer_metrics_async(info["log_metrics"], mode=mode, step=step)
    else:
      self.rl_engine.buffer_metrics(info["log_metrics"], mode=mode)
    return info["rewards"]

  # ---- the producer: dataloader micro-batches -> generated, scored, advantage-annotated examples ----
  #
  # Three small stages, each a generator over the previous one, run on the producer thread:
  #   _tagged_micro_batches : pulls dataloader items (skipping what a restored run already consumed),
  #                           repeats every prompt G times and stamps trajectory ids;
  #   _service_batches      : groups them until a rollout/log-prob service batch is full, runs
  #                           `_generate_and_compute_advantage` once per group and splits the result
  #                           back into the original micro-batches;
  #   _prepare_data         : decides WHEN results reach the trainer's queue (as they appear when rollout
  #                           and trainer run on different devices, else after the whole mini-batch) and
  #                           how often (`batch_repeat` passes, each freshly shuffled).
  def _tagged_micro_batches(self, iterator: Iterator[TrainingInputT], sample_repeat: int, mode: Mode, limit: int,
                            exhausted: List[bool]):
    train = mode == Mode.TRAIN
    if train and self._iter_steps < self._last_iter_step:
      behind = self._last_iter_step - self._iter_steps
      for _ in range(behind):            # a resumed run: these were trained on before the restart
        next(iterator, None)
      self._iter_steps = self._last_iter_step
      log.info("resumed: skipped %d already-consumed micro-batches", behind)
    taken = 0
    while limit <= 0 or taken < limit:
      with self.rl_engine.perf.span("data_loading"):
        raw = next(iterator, None)
      if raw is None:
        exhausted[0] = True
        return
      n_prompts = len(raw["prompts"])
      example = _repeat_tree(raw, sample_repeat)
      if "trajectory_ids" in example:
        raise ValueError("dataloader items must not carry 'trajectory_ids': the learner assigns them")
      example["trajectory_ids"] = self._compute_trajectory_ids(
          example, self._iter_steps if train else self._eval_iter_steps)
      for tid in example["trajectory_ids"]:
        self.rl_engine.buffer_metrics({"trajectory_ids": (tid, None)}, mode=mode)
      yield example, n_prompts, n_prompts * sample_repeat
      if train:
        self._iter_steps += 1
      else:
        self._eval_iter_steps += 1
      taken += 1

  def _service_batches(self, tagged, target_prompts: int, mode: Mode, drop_tail=lambda: False):
    group: List[TrainingInputT] = []
    sizes: List[int] = []
    prompts_in_group = 0

    def flush():
      if not group:
        return []
      whole = self._generate_and_compute_advantage(rl_utils.merge_micro_batches(group), mode)
      bounds = np.cumsum([0] + sizes)
      parts = [rl_utils.get_batch_slice(whole, slice(int(lo), int(hi))) for lo, hi in zip(bounds[:-1], bounds[1:])]
      group.clear()
      sizes.clear()
      return parts

    for example, n_prompts, n_rows in tagged:
      group.append(example)
      sizes.append(n_rows)
      prompts_in_group += n_prompts
      if prompts_in_group >= target_prompts:
        prompts_in_group = 0
        yield flush()
    if drop_tail():            # the dataloader ran dry inside a counted request: the caller discards it anyway
      return
    rest = flush()             # a last, smaller service batch
    if rest:
      yield rest

  def _process_accumulated_batches(self, micro_batches: List[TrainingInputT], micro_batch_sizes: List[int],
                                   mode: Mode) -> List[Any]:
    """One generate / advantage pass over several merged micro-batches, split back afterwards."""
    if not micro_batches:
      return []
    whole = self._generate_and_compute_advantage(rl_utils.merge_micro_batches(micro_batches), mode)
    bounds = np.cumsum([0] + list(micro_batch_sizes))
    return [rl_utils.get_batch_slice(whole, slice(int(lo), int(hi))) for lo, hi in zip(bounds[:-1], bounds[1:])]

  def _prepare_data(self, iterator: Iterator[TrainingInputT], proceed_num_steps: int, sample_repeat: int,
                    batch_repeat: int, service_target_batch_size: int, data_queue, async_loading: bool = False,
                    mode: Mode = Mode.TRAIN) -> None:
    """Fills `data_queue` with the examples of `proceed_num_steps` dataloader items (all of them when <= 0),
    each as a one-element list, and always ends it with `None` - also when the producer fails, so the
    consumer never waits forever. With a positive step count, a dataloader that runs dry first raises
    StopIteration (the epoch is over; what was collected is dropped)."""
    passes = 1 if mode == Mode.EVAL else batch_repeat
    stream_out = async_loading and mode == Mode.TRAIN      # hand results over while later ones are generated

    def deliver(examples: List[Any]) -> None:
      order: Iterable[int] = range(len(examples))
      if self._data_shuffle_rng is not None:
        order = self._data_shuffle_rng.permutation(len(examples))
      for i in order:
        data_queue.put([examples[i]])

    exhausted = [False]
    try:
      kept: List[Any] = []
      tagged = self._tagged_micro_batches(iterator, sample_repeat, mode, proceed_num_steps, exhausted)
      for produced in self._service_batches(tagged, service_target_batch_size, mode,
                                            drop_tail=lambda: exhausted[0] and proceed_num_steps > 0):
        if stream_out:
          deliver(produced)
        if not stream_out or passes > 1:
          kept.extend(produced)
      if exhausted[0] and proceed_num_steps > 0:
        raise StopIteration
      for _ in range(passes - 1 if stream_out else passes):
        deliver(kept)
    finally:
      data_queue.put(None)

  def _create_micro_batch_iterator(self, full_batch_iterator: Iterator[TrainingInputT],
                                   micro_batch_size: int) -> Iterator[TrainingInputT]:
    buffer: Dict[str, List[Any]] = {}
    for large in full_batch_iterator:
      for k, v in large.items():
        buf = buffer.setdefault(k, [])
        if isinstance(v, torch.Tensor):
          buf.extend(list(v))
        elif isinstance(v, np.ndarray):
          buf.extend(list(v))
        elif isinstance(v, (list, tuple)):
          buf.extend(v)
        else:
          buf.append(v)
      while buffer and len(next(iter(buffer.values()))) >= micro_batch_size:
        mb = {}
        for k in buffer:
          chunk = buffer[k][:micro_batch_size]
          buffer[k] = buffer[k][micro_batch_size:]
          if chunk and isinstance(chunk[0], torch.Tensor):
            mb[k] = torch.stack(chunk)
          elif chunk and isinstance(chunk[0], str):
            mb[k] = list(chunk)
          else:
            mb[k] = np.array(chunk)
        yield mb

  # ---- the loop ------------------------------------------------------------------------------------
  def train(self, train_ds: Iterable[TrainingInputT], eval_ds: Optional[Iterable[TrainingInputT]] = None,
            skip_jit: bool = False) -> None:
    it = iter(train_ds)
    first = next(it)
    full = len(first["prompts"])
    it = itertools.chain([first], it)
    tc = self._training_config
    mini = tc.mini_batch_size or full
    micro = tc.train_micro_batch_size or mini
    self._rollout_micro_batch_size = self._rollout_micro_batch_size or micro
    self._compute_logps_micro_batch_size = self._compute_logps_micro_batch_size or micro
    for v, n in [(self._rollout_micro_batch_size, "rollout_micro_batch_size"),
                 (self._compute_logps_micro_batch_size, "compute_logps_micro_batch_size"), (mini, "mini_batch_size")]:
      rl_utils.check_divisibility(v, full, n, f"full_batch_size={full}")
    ga = tc.get_with_default("gradient_accumulation_steps", 1)
    log.info("Training with full_batch_size=%d, mini_batch_size=%d, train_micro_batch_size=%d, "
             "rollout_micro_batch_size=%d, compute_logps_micro_batch_size=%d, grad_acc_steps=%d", full, mini, micro,
             self._rollout_micro_batch_size, self._compute_logps_micro_batch_size, ga)
    target = math.lcm(self._rollout_micro_batch_size, self._compute_logps_micro_batch_size)
    train_iterator = it if micro == full else self._create_micro_batch_iterator(it, micro)
    while True:
      try:
        with self.rl_engine.perf.span_group("global_step"):
          self._run_global_step(full, mini, target, ga, train_iterator, eval_ds, skip_jit)
          if self.should_sync_weights:
            with self.rl_engine.perf.span("weight_sync", self.rl_engine.perf.all_devices):
              self.rl_engine.sync_weights()
          else:
            self.rl_engine.global_steps += 1
        self.rl_engine.buffer_metrics(self.rl_engine.perf.export(), mode=Mode.TRAIN)
        self.rl_engine.buffer_metrics(self.rl_engine.perf_v2.export(), mode=Mode.TRAIN)
        if tc.max_steps is not None and self.rl_engine.actor_trainer.train_steps >= tc.max_steps:
          break
      except StopIteration:
        break
    self.rl_engine.close()

  def _run_global_step(self, full, mini, target, ga, train_iterator, eval_ds, skip_jit) -> None:
    for _ in range(full // mini):
      initial = self._iter_steps
      with self.rl_engine.perf.span_group("mini_batch_step"):
        self._run_mini_batch_step(initial, mini, target, ga, train_iterator, eval_ds, skip_jit)
      self._iter_steps = self.rl_engine.actor_trainer.iter_steps

  def _run_mini_batch_step(self, initial, mini, target, ga, train_iterator, eval_ds, skip_jit) -> None:
    with self.rl_engine.perf.span_group("micro_batch_steps"):
      self._run_all_micro_batch_steps(initial, mini, target, ga, train_iterator, eval_ds, skip_jit)

  def _run_all_micro_batch_steps(self, initial, mini, target, ga, train_iterator, eval_ds, skip_jit) -> None:
    train_q = queue_lib.SimpleDataQueue(maxsize=ga * self._num_iterations() + 1)
    eval_q = queue_lib.SimpleDataQueue(maxsize=0)
    future = self.executor.submit(
        self._prepare_data, iterator=train_iterator, proceed_num_steps=ga, sample_repeat=self._num_generations(),
        batch_repeat=self._num_iterations(), service_target_batch_size=target, data_queue=train_q,
        async_loading=self.can_enable_async_rollout, mode=Mode.TRAIN)

    def queue_iterator():
      while True:
        item = train_q.get(block=True)
        if item is None:
          break
        yield item

    gen = queue_iterator()
    tc = self._training_config
    if tc.max_seq_token_per_tpu is not None:
      mesh = self.rl_engine.cluster_config.role_to_mesh.get(Role.ACTOR)
      gen = rl_utils.pack_sequences(gen, tc.max_seq_token_per_tpu,
                                    sequences_per_update=mini * self._num_generations(),
                                    pad_id=self.rl_engine.rollout.pad_id(), pack_size=rl_utils.compute_pack_size(mesh),
                                    max_segments_per_packed_row=getattr(tc, "max_segments_per_packed_row", None))
    cur_eval = None
    while True:
      with sft_utils.time_measure(suppress_logging=True) as timer:
        cur_train = next(gen, None)
      if cur_train is None:
        break
      if self.can_enable_async_rollout:
        self.rl_engine.buffer_metrics({"actor_dequeue_time": (timer(), np.mean)}, mode=Mode.TRAIN)
      if eval_ds and not cur_eval and self.rl_engine.actor_trainer.train_steps % tc.eval_every_n_steps == 0:
        self._eval_iter_steps = 0
        self._prepare_data(iterator=iter(eval_ds), proceed_num_steps=-1, sample_repeat=self._num_generations(),
                           batch_repeat=1, service_target_batch_size=target, data_queue=eval_q, async_loading=False,
                           mode=Mode.EVAL)
        cur_eval = []
        while True:
          item = eval_q.get(block=True)
          if item is None:
            break
          cur_eval.extend(item)
      self.rl_engine.update_actor(cur_train, cur_eval, skip_jit)
      if hasattr(self.rl_engine, "_critic_trainer"):
        self.rl_engine.update_critic(cur_train, cur_eval, skip_jit)
    future.result()       # re-raises a producer exception in the training thread

  @property
  def rl_cluster(self):
    return self.rl_engine

  @rl_cluster.setter
  def rl_cluster(self, value):
    self.rl_engine = value
