"""Asynchronous producer / consumer RL learner for multi-turn agents
(tunix/rl/agentic/agentic_rl_learner.py:67-1254).

A dedicated asyncio loop thread (executor of `max_concurrency + 1` threads) runs the rollout
side: prompts are fed through a queue that is prefilled with `off_policy_steps + 1` batches, a
`RolloutOrchestrator` streams finished groups of `num_generations` episodes, each group is
turned into `TrainExample`s by the algorithm (`_process_results`) and put on the training
queue. The calling thread consumes micro-batches and trains while later rollouts continue.
After every full batch: `num_iterations - 1` further passes over the batch, a weight sync
under the `RolloutSyncLock` (episodes in flight finish first, new ones wait), the policy
version is bumped and the next prompt batch is released.
"""
from __future__ import annotations

import abc
import asyncio
import contextlib
import copy
import dataclasses
import itertools
import logging
import queue
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from typing import Any, Dict, Generic, Iterable, Iterator, List, Optional, Sequence, Set, Type, TypeVar

import numpy as np
import torch

from ...common.datatypes import Mode, Role
from .. import algorithm_config as algo_config_lib, common, function_registry, utils as rl_utils
from ..queue import data_queue as queue_lib
from . import utils as agentic_utils
from .agents import base_agent, model_agent
from .environments import base_environment, task_environment
from .pipeline import rollout_orchestrator
from .trajectory import trajectory_collect_engine

TrainingInputT = Dict[str, Any]


@dataclasses.dataclass(frozen=True)
class TrainExample(common.TrainExample):
  policy_version: Any = None


@dataclasses.dataclass(kw_only=True)
class AgenticRLConfig(algo_config_lib.AlgorithmConfig):
  system_prompt: str = ""
  reward_manager: str = "agentic-sequence-level"
  max_response_length: int = 1024
  max_concurrency: int = 32
  off_policy_steps: int = 0
  num_generations: int = 1
  num_iterations: int = 1
  episode_timeout: float = 1800.0
  filter_statuses: Optional[Set] = None
  overlong_filter: bool = False
  use_rollout_logps: bool = True


TConfig = TypeVar("TConfig", bound=AgenticRLConfig)


class _QueueAsyncIter:
  """Async view of a thread queue; `None` ends the iteration."""

  def __init__(self, q: "queue.Queue", loop: asyncio.AbstractEventLoop):
    self.q, self.loop = q, loop

  def __aiter__(self):
    return self

  async def __anext__(self):
    item = await self.loop.run_in_executor(None, self.q.get)
    if item is None:
      raise StopAsyncIteration
    return item


def _batch_len(batch: TrainingInputT) -> int:
  return len(next(iter(batch.values())))


def _cat_examples(examples: Sequence[Any]):
  """Concatenates dataclass examples on the batch axis (None fields stay None)."""
  first = examples[0]
  if len(examples) == 1:
    return first
  kw = {}
  for f in dataclasses.fields(first):
    vals = [getattr(e, f.name) for e in examples]
    v0 = vals[0]
    if isinstance(v0, torch.Tensor) and v0.dim() > 0:
      kw[f.name] = torch.cat(vals, 0)
    elif isinstance(v0, np.ndarray) and v0.ndim > 0:
      kw[f.name] = np.concatenate(vals, 0)
    else:
      kw[f.name] = v0
  return type(first)(**kw)


def _slice_example(ex, sl: slice, n_total: int):
  kw = {}
  for f in dataclasses.fields(ex):
    v = getattr(ex, f.name)
    kw[f.name] = v[sl] if hasattr(v, "shape") and len(v.shape) > 0 and v.shape[0] == n_total else v
  return type(ex)(**kw)


class AgenticRLLearner(abc.ABC, Generic[TConfig]):
  def __init__(self, rl_engine=None, algo_config: TConfig = None, reward_fns=None, chat_parser: Any = None,
               metric_fns: Optional[Sequence[Any]] = None,
               agent_class: Type[base_agent.ConversationAgentBase] = model_agent.ModelAgent,
               agent_kwargs: Optional[Dict[str, Any]] = None,
               env_class: Type[base_environment.BaseTaskEnv] = task_environment.TaskEnvironment,
               env_kwargs: Optional[Dict[str, Any]] = None, rl_cluster=None):
    self.rl_engine = rl_engine if rl_engine is not None else rl_cluster
    self.algo_config = algo_config
    self._validate_rollout_config()
    self.reward_manager = function_registry.get_reward_manager(algo_config.reward_manager)(
        reward_fns=reward_fns, algo_config=algo_config)
    self.metric_fns = list(metric_fns or [])
    eng = self.rl_engine
    eng.actor_trainer.is_managed_externally = True
    if getattr(eng, "_critic_trainer", None) is not None:
      eng.critic_trainer.is_managed_externally = True
    self.agent_class, self.agent_kwargs = agent_class, agent_kwargs or {}
    self.env_class, self.env_kwargs = env_class, env_kwargs or {}
    self._training_config = eng.cluster_config.training_config
    eng.global_steps = eng.actor_trainer.restored_global_step()
    self._iter_steps = eng.actor_trainer.iter_steps
    self._last_eval_train_step = -1
    self.should_sync_weights = getattr(eng.rollout, "holds_own_weights", False) or \
        not rl_utils.is_sharing_weights(eng.actor_trainer.model, eng.rollout.model())
    r2m = eng.cluster_config.role_to_mesh
    self.can_enable_async_rollout = r2m[Role.ACTOR] != r2m[Role.ROLLOUT]
    self._compute_logps_micro_batch_size = self._training_config.compute_logps_micro_batch_size or 1
    self.chat_parser = chat_parser
    self.tokenizer = eng.tokenizer
    self.policy_version = eng.global_steps
    self._rollout_sync_lock = agentic_utils.RolloutSyncLock()
    self._background_tasks: Set[asyncio.Task] = set()
    self._full_batch_size = 0
    self._process_in_consumer = False
    self._train_rewards: List[float] = []
    self._eval_rewards: List[float] = []
    self._rewards_lock = threading.Lock()
    self._global_step_start = time.time()
    # the rollout side lives on its own event loop thread
    ready: "queue.Queue" = queue.Queue()

    try:
      home = next(self.rl_engine.actor_trainer.model.parameters()).device
    except (StopIteration, AttributeError):
      home = None

    def bind():     # helper threads start on CUDA device 0; they must use this rank's GPU
      if home is not None and home.type == "cuda":
        torch.cuda.set_device(home)

    def run_loop():
      bind()
      loop = asyncio.new_event_loop()
      asyncio.set_event_loop(loop)
      loop.set_default_executor(ThreadPoolExecutor(max_workers=algo_config.max_concurrency + 1, initializer=bind))
      ready.put(loop)
      loop.run_forever()
    self._loop_thread = threading.Thread(target=run_loop, daemon=True, name="agentic-rollout-loop")
    self._loop_thread.start()
    self.loop: asyncio.AbstractEventLoop = ready.get()

  # ---- configuration checks ------------------------------------------------------------------
  def _validate_rollout_config(self) -> None:
    rc = self.rl_engine.cluster_config.rollout_config
    for mode, cfg in (rc.items() if isinstance(rc, dict) else [("train", rc)]):
      if cfg.max_tokens_to_generate != self.algo_config.max_response_length:
        raise ValueError(f"RolloutConfig ({mode}) max_tokens_to_generate ({cfg.max_tokens_to_generate}) must match "
                         f"AgenticRLConfig max_response_length ({self.algo_config.max_response_length}). Please align "
                         "these configurations before initializing RLEngine.")
      if self.algo_config.use_rollout_logps and not cfg.return_logprobs:
        raise ValueError(f"RolloutConfig ({mode}) must have return_logprobs=True for AgenticRLLearner when "
                         "use_rollout_logps=True. Please set this before initializing RLEngine.")
      if self.rl_engine.cluster_config.rollout_engine == "vllm" and not cfg.rollout_vllm_server_mode:
        raise ValueError(f"RolloutConfig ({mode}) must have rollout_vllm_server_mode set to True for "
                         "AgenticRLLearner if using vLLM engine. Please set this before initializing RLEngine.")

  # ---- rewards -------------------------------------------------------------------------------
  def _compute_rewards(self, prompts: List[str], completions: List[str], mode: Mode,
                       expected_step: Optional[int] = None, **kwargs) -> np.ndarray:
    if "mode" in kwargs:
      raise ValueError(f"kwargs already contains mode as a key: {kwargs}")
    kwargs["mode"] = str(mode)
    info = self.reward_manager(prompts=prompts, completions=completions, **kwargs)
    self.rl_engine.buffer_metrics_async(info["log_metrics"], mode=mode, step=expected_step or 0)
    rewards = np.asarray(info["rewards"])
    with self._rewards_lock:
      window = self._train_rewards if mode == Mode.TRAIN else self._eval_rewards
      window.extend(rewards.tolist())
      if mode == Mode.TRAIN and self._full_batch_size > 0:
        cap = self._full_batch_size * self.algo_config.num_generations
        del window[:max(0, len(window) - cap)]
    return info["rewards"]

  # ---- rollout side --------------------------------------------------------------------------
  @staticmethod
  def _single_examples(batches: Iterable[TrainingInputT]) -> Iterator[TrainingInputT]:
    """Splits batches {key: [B, ...]} into one-example dicts {key: array of 1}."""
    for batch in batches:
      cols = {k: (list(np.asarray(v).reshape(len(v), -1)[:, 0]) if isinstance(v, (np.ndarray, torch.Tensor))
                  and np.asarray(v).ndim > 1 else list(v)) if isinstance(v, (list, tuple, np.ndarray, torch.Tensor))
              else [v] for k, v in batch.items()}
      n = len(next(iter(cols.values())))
      for i in range(n):
        yield {k: np.array(c[i:i + 1]) for k, c in cols.items()}

  def _create_agent_env_pair(self, single_example: TrainingInputT, group_id: int, pair_index: int):
    agent = self.agent_class(**{"system_prompt": self.algo_config.system_prompt, **self.agent_kwargs})
    assert "group_id" not in self.env_kwargs and "pair_index" not in self.env_kwargs
    env = self.env_class(single_example, **{"group_id": group_id, "pair_index": pair_index, **self.env_kwargs})
    return agent, env

  def _model_call(self, chat_lists, env: Any = None, max_generation_steps: Optional[int] = None):
    if env is not None:
      env.task["policy_version"] = self.policy_version
    if self.chat_parser:
      chat_lists = self.chat_parser.parse(messages=chat_lists, add_generation_prompt=True, is_first_msg=True)
    tags = {}
    extra = getattr(env, "extra_kwargs", None) or {}
    if "group_id" in extra:
      tags["group_id"] = extra["group_id"]
      if self._full_batch_size > 0:
        tags["step"] = extra["group_id"] // self._full_batch_size
    if "pair_index" in extra:
      tags["pair_index"] = extra["pair_index"]
    return self.rl_engine.generate(prompts=[chat_lists], apply_chat_template=not self.chat_parser, mode=Mode.TRAIN,
                                   trace_tags=tags, max_generation_steps=max_generation_steps)

  def _build_orchestrator(self) -> rollout_orchestrator.RolloutOrchestrator:
    cfg = self.algo_config
    return rollout_orchestrator.RolloutOrchestrator(
        engine_cls=trajectory_collect_engine.TrajectoryCollectEngine,
        engine_kwargs=dict(model_call=self._model_call, tokenizer=self.tokenizer, chat_parser=self.chat_parser,
                           timeout=cfg.episode_timeout, max_response_length=cfg.max_response_length,
                           overlong_filter=cfg.overlong_filter, filter_statuses=cfg.filter_statuses,
                           perf_v2=getattr(self.rl_engine, "perf_v2", None)),
        max_concurrency=cfg.max_concurrency, rollout_sync_lock=self._rollout_sync_lock)

  async def _orchestrator_producer(self, orchestrator, prompt_iterator, num_generations: int = 1,
                                   collect_mode: str = "Token"):
    """Yields groups (lists of `TrajectoryItem`) of `num_generations` episodes per prompt."""
    is_async = hasattr(prompt_iterator, "__aiter__")
    loop = asyncio.get_running_loop()

    async def pairs():
      group_id = self.rl_engine.global_steps * self._full_batch_size

      async def expand(example):
        return await asyncio.gather(*[loop.run_in_executor(None, self._create_agent_env_pair, copy.deepcopy(example),
                                                           group_id, j) for j in range(num_generations)])
      if is_async:
        async for example in prompt_iterator:
          for pair in await expand(example):
            yield pair
          group_id += 1
      else:
        for example in prompt_iterator:
          for pair in await expand(example):
            yield pair
          group_id += 1

    producer = asyncio.create_task(orchestrator.run_producers_from_stream(
        pairs_stream=pairs(), group_size=self.algo_config.num_generations,
        group_key_fn=lambda i, env, traj: env.extra_kwargs["group_id"], collect_mode=collect_mode))
    await asyncio.sleep(0)
    gen = orchestrator.yield_batches(batch_size=self.algo_config.num_generations)
    try:
      async with contextlib.aclosing(gen) as stream:
        async for group in stream:
          if group:
            yield group
      if producer.done() and not producer.cancelled() and producer.exception() is not None:
        raise producer.exception()
    finally:
      if not producer.done():
        producer.cancel()

        async def drain():
          with contextlib.suppress(asyncio.CancelledError, Exception):
            await producer
        t = asyncio.create_task(drain())
        self._background_tasks.add(t)
        t.add_done_callback(self._background_tasks.discard)

  def _batch_to_train_example(self, batch_results: List[Any], mode: Mode) -> List[TrainExample]:
    if mode == Mode.TRAIN:
      expected_step = batch_results[0].group_id // max(self._full_batch_size, 1)
    else:
      expected_step = self.rl_engine.global_steps
    return self._process_results(trajectories=batch_results, mode=mode, expected_step=expected_step)

  def _compute_packed_logps(self, example):
    return example

  @abc.abstractmethod
  def _process_results(self, trajectories: List[Any], mode: Mode = Mode.TRAIN,
                       expected_step: Optional[int] = None) -> List[TrainExample]: ...

  def _generate_and_compute_advantage(self, training_input, mode: Mode = Mode.TRAIN):
    raise NotImplementedError("_generate_and_compute_advantage is not used in AgenticRLLearner")

  def _num_iterations(self) -> int:
    return self.algo_config.num_iterations

  def _num_generations(self) -> int:
    return self.algo_config.num_generations

  async def _producer(self, orchestrator, prompt_queue: "queue.Queue", train_data_queue) -> None:
    """Prompt queue -> episodes -> TrainExamples -> training queue; `None` marks the end, an
    exception object is forwarded so that the consumer re-raises it."""
    loop = asyncio.get_running_loop()

    async def prompts():
      async for batch in _QueueAsyncIter(prompt_queue, loop):
        for example in self._single_examples([batch]):
          yield example
    try:
      async for group in self._orchestrator_producer(orchestrator, prompts(), self.algo_config.num_generations, "Token"):
        if self._process_in_consumer:
          train_data_queue.put(group)
        else:
          train_data_queue.put(await loop.run_in_executor(None, self._batch_to_train_example, group, Mode.TRAIN))
    except BaseException as e:  # the consumer must not wait forever
      train_data_queue.put(e)
      raise
    finally:
      train_data_queue.put(None)

  def _data_consumer_batch_generator(self, q, batch_size: int) -> Iterator[List[Any]]:
    """Groups of examples from the queue, `batch_size` groups at a time."""
    buf: List[Any] = []
    while True:
      item = q.get(block=True)
      if isinstance(item, BaseException):
        raise item
      if item is None:
        if buf:
          yield buf
        return
      buf.append(item)
      if len(buf) == batch_size:
        yield buf
        buf = []

  # ---- training side -------------------------------------------------------------------------
  def _put_prompts_to_queue(self, prompt_queue: "queue.Queue", batch: TrainingInputT) -> None:
    tc = self._training_config
    if tc.max_steps and self.rl_engine.global_steps >= tc.max_steps:
      prompt_queue.put(None)
    elif _batch_len(batch) != self._full_batch_size:
      logging.warning("partial batch %d vs %d detected. The rest of the batch will be skipped.", _batch_len(batch),
                      self._full_batch_size)
      prompt_queue.put(None)
    else:
      prompt_queue.put(batch)

  def _feed_next(self, it: Iterator[TrainingInputT], prompt_queue: "queue.Queue") -> None:
    try:
      self._put_prompts_to_queue(prompt_queue, next(it))
    except StopIteration:
      prompt_queue.put(None)

  def _filter_outdated_offpolicy_examples(self, examples: List[TrainExample]) -> List[TrainExample]:
    keep = []
    for ex in examples:
      pv = ex.policy_version
      if pv is not None and (int(pv[0]) == -1 or self.policy_version - int(pv[0]) <= self.algo_config.off_policy_steps):
        keep.append(ex)
    if not keep:
      logging.warning("all examples of a micro-batch were older than off_policy_steps=%d and were dropped",
                      self.algo_config.off_policy_steps)
    return keep

  def _run_eval(self, eval_prompts: List[TrainingInputT]) -> List[TrainExample]:
    orchestrator = self._build_orchestrator()

    async def run():
      out: List[TrainExample] = []
      async for group in self._orchestrator_producer(orchestrator, eval_prompts, self._num_generations()):
        out.extend(self._batch_to_train_example(group, Mode.EVAL))
      return out
    return asyncio.run_coroutine_threadsafe(run(), self.loop).result()

  def _log_step(self, last_batch, step_time: float, did_eval: bool) -> None:
    with self._rewards_lock:
      tr = np.asarray(self._train_rewards, np.float32)
      ev = np.asarray(self._eval_rewards, np.float32)
      self._train_rewards.clear()
      if did_eval:
        self._eval_rewards.clear()
    adv = np.asarray(torch.as_tensor(last_batch.advantages).float().cpu())
    cm = np.asarray(torch.as_tensor(last_batch.completion_mask).float().cpu())
    msg = (f"[step {self.rl_engine.global_steps}] train_reward={tr.mean() if tr.size else float('nan'):.3f} "
           f"train_solve={(tr > 0.1).mean() if tr.size else float('nan'):.3f} n={tr.size} "
           f"adv_abs_mean={np.abs(adv).mean() if adv.size else float('nan'):.3f} "
           f"compl_len={cm.sum(-1).mean() if cm.size else 0.0:.1f} time={step_time:.1f}s")
    if did_eval and ev.size:
      msg += f" eval_reward={ev.mean():.3f} eval_solve={(ev > 0.1).mean():.3f} eval_n={ev.size}"
    logging.info(msg)

  def train(self, train_dataset: Iterable[TrainingInputT], eval_dataset: Optional[Iterable[TrainingInputT]] = None,
            skip_jit: bool = False) -> None:
    eng, tc, cfg = self.rl_engine, self._training_config, self.algo_config
    it = iter(train_dataset)
    for _ in range(eng.global_steps):         # resume: skip what earlier runs consumed
      if next(it, None) is None:
        logging.warning("Train dataset exhausted while skipping batches.")
        eng.close()
        return
    first = next(it, None)
    if first is None:
      logging.warning("Training dataset is empty.")
      eng.close()
      return
    full = self._full_batch_size = _batch_len(first)
    mini = tc.mini_batch_size or full
    micro = tc.train_micro_batch_size or mini
    packing = tc.max_seq_token_per_tpu is not None
    process_in_consumer = False
    if self._compute_logps_micro_batch_size > 1 and not packing:
      if self._compute_logps_micro_batch_size != micro:
        raise ValueError(f"compute_logps_micro_batch_size ({self._compute_logps_micro_batch_size}) must be equal to "
                         f"train_micro_batch_size ({micro})")
      process_in_consumer = True
    for v, n in ((self._compute_logps_micro_batch_size, "compute_logps_micro_batch_size"), (mini, "mini_batch_size")):
      rl_utils.check_divisibility(v, full, n, "full_batch_size")
    grad_acc = tc.get_with_default("gradient_accumulation_steps", 1)
    data_it = itertools.chain([first], it)
    eval_prompts = list(self._single_examples(eval_dataset)) if eval_dataset else []

    train_q = queue_lib.SimpleDataQueue(maxsize=0)
    prompt_q: "queue.Queue" = queue.Queue()
    for _ in range(cfg.off_policy_steps + 1):
      self._feed_next(data_it, prompt_q)
    orchestrator = self._build_orchestrator()
    # with `process_in_consumer` the producer forwards raw groups and they are converted on the
    # training thread, `micro` groups at a time, so the log-prob passes run at that batch size
    self._process_in_consumer = process_in_consumer
    producer_future = asyncio.run_coroutine_threadsafe(self._producer(orchestrator, prompt_q, train_q), self.loop)
    gen = self._data_consumer_batch_generator(train_q, micro)
    if process_in_consumer:
      def convert(raw):
        for groups in raw:
          yield [self._batch_to_train_example([t for g in groups for t in g], Mode.TRAIN)]
      gen = convert(gen)
    if packing:
      gen = rl_utils.pack_sequences(gen, tc.max_seq_token_per_tpu, sequences_per_update=mini * self._num_generations(),
                                    pack_size=rl_utils.compute_pack_size(eng.cluster_config.role_to_mesh[Role.ACTOR]),
                                    max_segments_per_packed_row=getattr(tc, "max_segments_per_packed_row", None))
    updates_per_full = full // mini
    updates_since_sync = micro_steps = 0
    did_eval = False
    chunks: List[Any] = []
    merged = None
    has_critic = getattr(eng, "_critic_trainer", None) is not None
    try:
      for micro_batch in gen:
        if tc.max_steps and eng.global_steps >= tc.max_steps:
          prompt_q.put(None)
          break
        self._iter_steps += 1
        flat = [e for group in micro_batch for e in (group if isinstance(group, (list, tuple)) else [group])]
        merged = _cat_examples(flat)
        is_packed = getattr(merged, "segment_ids", None) is not None
        if is_packed:
          merged = self._compute_packed_logps(merged)
          seg = np.asarray(torch.as_tensor(merged.segment_ids).cpu())
          eng.buffer_metrics_async({"packing/dummy_ratio": (float((seg == 0).mean()), np.mean),
                                    "packing/seqs_per_pack": (float(seg.max(-1).mean()), np.mean)},
                                   mode=Mode.TRAIN, step=eng.global_steps)
          step_chunks = [merged]
        else:
          per = micro * cfg.num_generations
          n = merged.completion_ids.shape[0]
          step_chunks = [_slice_example(merged, slice(i, i + per), n) for i in range(0, n, per)] if n > per else [merged]
        chunks.extend(step_chunks)
        eval_ds = None
        if updates_since_sync == 0 and eval_prompts:
          cur = eng.actor_trainer.train_steps
          if cur % tc.eval_every_n_steps == 0 and cur != self._last_eval_train_step:
            self._last_eval_train_step = cur
            eval_ds = self._run_eval(eval_prompts)
            did_eval = True
        eng.update_actor(step_chunks, eval_ds, skip_jit)
        if has_critic:
          eng.update_critic(step_chunks, eval_ds, skip_jit)
        if is_packed:
          is_update = bool(np.asarray(torch.as_tensor(merged.is_update_step).cpu()).item())
        else:
          micro_steps += len(step_chunks)
          is_update = micro_steps % grad_acc == 0
        if is_update:
          updates_since_sync += 1
        if updates_since_sync != updates_per_full:
          continue
        # ---- one full batch has been trained on ----
        for _ in range(1, self._num_iterations()):
          self._iter_steps += len(chunks)
          eng.update_actor(chunks, None, skip_jit)
          if has_critic:
            eng.update_critic(chunks, None, skip_jit)
        chunks = []
        step_time = time.time() - self._global_step_start
        self._log_step(merged, step_time, did_eval)
        eng.buffer_metrics_async({"perf/global_step_time": (step_time, np.mean)}, mode=Mode.TRAIN, step=eng.global_steps)
        if self.should_sync_weights:
          with self._rollout_sync_lock.weight_sync():
            eng.sync_weights()                      # advances global_steps
            self.policy_version += 1
            self._feed_next(data_it, prompt_q)
        else:
          eng.global_steps += 1
          self.policy_version += 1
          self._feed_next(data_it, prompt_q)
        updates_since_sync = 0
        did_eval = False
        self._global_step_start = time.time()
    finally:
      prompt_q.put(None)
    try:
      producer_future.result(timeout=60)
    except (asyncio.CancelledError, TimeoutError):
      producer_future.cancel()
    eng.close()
