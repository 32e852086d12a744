"""Sampler backed by an in-process vLLM engine (tunix/generate/vllm_sampler.py).

The engine is created from a Hugging Face style directory: either `VllmConfig.model_path`, or an
export of the trainer's model written once at start-up (`config.json` derived from our
`ModelConfig`, weights through `models.safetensors_saver`). Weight sync (`update_params`) streams
the trainer's parameters, renamed to Hugging Face names and split where we fuse projections, into
the engine's `load_weights`. Requests can run in two ways:

* batch mode (default): one `LLM.generate` call per rollout;
* server mode (`rollout_vllm_server_mode`): a driver thread owns the engine and drains a queue
  of requests, submitting them as soon as `submission_threshold` are waiting or
  `submission_timeout_s` has passed, so concurrent producers (agentic rollouts) share batches.

Everything vLLM-specific is imported lazily; the module imports without the package.
"""
from __future__ import annotations

import dataclasses
import json
import os
import queue
import tempfile
import threading
import time
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import base_sampler, tokenizer_adapter

_ARCH = {"llama3": ("LlamaForCausalLM", "llama"), "qwen2": ("Qwen2ForCausalLM", "qwen2"),
         "qwen3": ("Qwen3ForCausalLM", "qwen3"), "qwen3_moe": ("Qwen3MoeForCausalLM", "qwen3_moe"),
         "gemma": ("GemmaForCausalLM", "gemma"), "gemma2": ("Gemma2ForCausalLM", "gemma2"),
         "gemma3": ("Gemma3ForCausalLM", "gemma3_text")}


def hf_config_dict(cfg) -> Dict[str, Any]:
  """A Hugging Face `config.json` for one of our decoder configs."""
  fam = str(getattr(cfg, "family", "llama3"))
  if fam == "qwen3" and getattr(cfg, "is_moe", False):
    fam = "qwen3_moe"
  if fam == "gemma" and getattr(cfg, "use_post_ffw_norm", False):
    fam = "gemma2"
  arch, model_type = _ARCH.get(fam, _ARCH["llama3"])
  d = {
      "architectures": [arch], "model_type": model_type, "vocab_size": cfg.vocab_size, "hidden_size": cfg.embed_dim,
      "intermediate_size": cfg.hidden_dim, "num_hidden_layers": cfg.num_layers,
      "num_attention_heads": cfg.num_heads, "num_key_value_heads": cfg.num_kv_heads, "head_dim": cfg.head_dim,
      "rms_norm_eps": cfg.norm_eps, "rope_theta": cfg.rope_theta, "tie_word_embeddings": bool(cfg.weight_tying),
      "max_position_embeddings": int(getattr(cfg, "max_position", None) or 32768),
      "torch_dtype": str(cfg.dtype).replace("torch.", ""), "attention_bias": bool(getattr(cfg, "qkv_bias", False)),
      "hidden_act": "silu" if cfg.activation == "silu" else "gelu_pytorch_tanh",
  }
  if getattr(cfg, "is_moe", False):
    d.update(num_experts=cfg.num_experts, num_experts_per_tok=cfg.num_experts_per_tok,
             moe_intermediate_size=cfg.moe_hidden_dim, norm_topk_prob=bool(cfg.norm_topk_prob),
             decoder_sparse_step=1, mlp_only_layers=[])
  if getattr(cfg, "sliding_window_size", None):
    d["sliding_window"] = cfg.sliding_window_size
  if getattr(cfg, "attn_logits_soft_cap", None):
    d["attn_logit_softcapping"] = cfg.attn_logits_soft_cap
  if getattr(cfg, "final_logit_softcap", None):
    d["final_logit_softcapping"] = cfg.final_logit_softcap
  if getattr(cfg, "query_pre_attn_scalar", None):
    d["query_pre_attn_scalar"] = cfg.query_pre_attn_scalar
  return d


def _in_process_engine() -> None:
  """Weight sync hands device tensors to the engine's model without a copy through a pipe, which needs the
  engine core in this process: vLLM's switch for that is an environment variable read at engine start-up.
  A value the user has set wins."""
  os.environ.setdefault("VLLM_ENABLE_V1_MULTIPROCESSING", "0")


@dataclasses.dataclass
class VllmConfig:
  model_path: Optional[str] = None
  max_model_len: int = 2048
  tensor_parallel_size: int = 1
  data_parallel_size: int = 1
  expert_parallel_size: int = 1
  hbm_utilization: float = 0.2
  init_with_random_weights: bool = True
  seed: int = 0
  server_mode: bool = False
  request_timeout_s: Optional[float] = 1800.0     # server mode: how long a caller waits for one request
  submission_threshold: int = 0
  submission_timeout_s: float = 0.0
  logprobs_mode: str = "processed_logprobs"
  max_num_batched_tokens: Optional[int] = None
  max_num_seqs: Optional[int] = None
  lora_config: Optional[Dict[str, Any]] = None
  engine_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)
  sampling_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)

  @classmethod
  def from_rollout_config(cls, rc, mesh=None) -> "VllmConfig":
    tp = rc.tensor_parallel_size if rc.tensor_parallel_size and rc.tensor_parallel_size > 0 else 1
    dp = rc.data_parallel_size if rc.data_parallel_size and rc.data_parallel_size > 0 else 1
    if mesh is not None and rc.tensor_parallel_size in (None, -1):
      tp = max(1, getattr(mesh, "size", 1) // dp)
    return cls(
        model_path=rc.rollout_vllm_model_version or None, max_model_len=int(rc.kv_cache_size),
        tensor_parallel_size=tp, data_parallel_size=dp, expert_parallel_size=rc.expert_parallel_size or 1,
        hbm_utilization=rc.rollout_vllm_hbm_utilization,
        init_with_random_weights=rc.rollout_vllm_init_with_random_weights, seed=rc.seed or 0,
        server_mode=rc.rollout_vllm_server_mode,
        submission_threshold=rc.rollout_vllm_server_mode_submission_threshold,
        submission_timeout_s=rc.rollout_vllm_server_mode_submission_timeout_s,
        logprobs_mode=rc.rollout_vllm_logprobs_mode, max_num_batched_tokens=rc.rollout_vllm_max_num_batched_tokens,
        max_num_seqs=rc.rollout_vllm_max_num_seqs, lora_config=rc.rollout_vllm_lora_config,
        engine_kwargs=dict(rc.rollout_vllm_kwargs or {}), sampling_kwargs=dict(rc.rollout_vllm_sampling_kwargs or {}))

  def engine_args(self, model_dir: str) -> Dict[str, Any]:
    args = dict(model=model_dir, tokenizer=None, skip_tokenizer_init=True, max_model_len=self.max_model_len,
                tensor_parallel_size=self.tensor_parallel_size, gpu_memory_utilization=self.hbm_utilization,
                seed=self.seed, enforce_eager=False, logprobs_mode=self.logprobs_mode)
    if self.data_parallel_size > 1:
      args["data_parallel_size"] = self.data_parallel_size
    if self.expert_parallel_size > 1:
      args["enable_expert_parallel"] = True
    if self.init_with_random_weights:
      args["load_format"] = "dummy"
    if self.max_num_batched_tokens:
      args["max_num_batched_tokens"] = self.max_num_batched_tokens
    if self.max_num_seqs:
      args["max_num_seqs"] = self.max_num_seqs
    if self.lora_config:
      args.update(enable_lora=True, max_lora_rank=int(self.lora_config.get("rank", 16)))
    args.update(self.engine_kwargs)
    return args


@dataclasses.dataclass
class _Request:
  prompt_ids: List[List[int]]
  params: Any
  done: threading.Event = dataclasses.field(default_factory=threading.Event)
  result: Any = None
  error: Optional[BaseException] = None


class GenerateBatchDriver:
  """Owns an object that only offers a blocking `generate` on one thread; batches queued requests by count or age
  before submitting them. Engines that can be stepped get `vllm_async_driver.VLLMInProcessDriver` instead."""

  def __init__(self, llm, threshold: int = 0, timeout_s: float = 0.0):
    self._llm = llm
    self._threshold = max(int(threshold), 1)
    self._timeout = float(timeout_s)
    self._q: "queue.Queue[Optional[_Request]]" = queue.Queue()
    self._thread = threading.Thread(target=self._loop, daemon=True, name="vllm-driver")
    self._thread.start()

  def submit(self, prompt_ids: List[List[int]], params) -> _Request:
    req = _Request(prompt_ids, params)
    self._q.put(req)
    return req

  def _loop(self) -> None:
    while True:
      first = self._q.get()
      if first is None:
        return
      batch = [first]
      deadline = time.monotonic() + self._timeout
      while len(batch) < self._threshold:
        left = deadline - time.monotonic()
        if left <= 0:
          break
        try:
          nxt = self._q.get(timeout=left)
        except queue.Empty:
          break
        if nxt is None:
          self._q.put(None)
          break
        batch.append(nxt)
      try:
        flat = [{"prompt_token_ids": p} for r in batch for p in r.prompt_ids]
        params = [r.params for r in batch for _ in r.prompt_ids]
        outs = self._llm.generate(flat, params, use_tqdm=False)
        pos = 0
        for r in batch:
          r.result = outs[pos:pos + len(r.prompt_ids)]
          pos += len(r.prompt_ids)
      except BaseException as e:  # pylint: disable=broad-exception-caught
        for r in batch:
          r.error = e
      for r in batch:
        r.done.set()

  def close(self) -> None:
    self._q.put(None)
    self._thread.join(timeout=5.0)


class VllmSampler(base_sampler.BaseSampler):

  def __init__(self, tokenizer: Any, config: VllmConfig, model: Optional[torch.nn.Module] = None, llm: Any = None):
    """`llm` injects a ready engine (tests, or an engine shared between samplers)."""
    self.tokenizer = tokenizer if isinstance(tokenizer, tokenizer_adapter.TokenizerAdapter) else \
        tokenizer_adapter.TokenizerAdapter(tokenizer)
    self.config = config
    self._model = model
    self._tmp = None
    if llm is None:
      _in_process_engine()
      import vllm
      llm = vllm.LLM(**config.engine_args(self._model_dir()))
    self.llm = llm
    self._driver = self._step_driver = None
    if config.server_mode:
      engine = getattr(llm, "llm_engine", None)
      if all(hasattr(engine, m) for m in ("add_request", "step", "has_unfinished_requests", "abort_request")):
        from . import vllm_async_driver
        self._step_driver = vllm_async_driver.VLLMInProcessDriver(
            engine, submission_threshold=config.submission_threshold, submission_timeout_s=config.submission_timeout_s)
      else:
        self._driver = GenerateBatchDriver(llm, config.submission_threshold, config.submission_timeout_s)
    if model is not None and not config.model_path and config.init_with_random_weights:
      self.update_params(dict(model.named_parameters()))

  # -- engine start-up ---------------------------------------------------------------------
  def _model_dir(self) -> str:
    if self.config.model_path:
      return self.config.model_path
    if self._model is None:
      raise ValueError("VllmSampler needs `config.model_path` or a model to export")
    self._tmp = tempfile.TemporaryDirectory(prefix="tunix_b200_vllm_")
    d = self._tmp.name
    with open(os.path.join(d, "config.json"), "w", encoding="utf-8") as f:
      json.dump(hf_config_dict(self._model.config), f)
    if not self.config.init_with_random_weights:
      from ..models import safetensors_io, safetensors_saver
      safetensors_io.save_file(safetensors_saver.to_hf_state(self._model), os.path.join(d, "model.safetensors"))
    return d

  @property
  def transformer(self):
    return self._model

  @property
  def transformer_state(self):
    return dict(self._model.named_parameters()) if self._model is not None else {}

  def tokenize(self, input_string: str) -> np.ndarray:
    ids = list(self.tokenizer.encode(input_string))
    bos = self.tokenizer.bos_id()
    if bos is not None and bos != 0 and (not ids or ids[0] != bos):
      ids = [bos] + ids
    return np.asarray(ids, dtype=np.int64)

  # -- weight sync ---------------------------------------------------------------------------
  def hf_named_weights(self, params: Dict[str, torch.Tensor]) -> Iterable[Tuple[str, torch.Tensor]]:
    """Trainer parameters under Hugging Face names (fused projections split, experts unstacked)."""
    from . import mappings
    cfg = self._model.config if self._model is not None else None
    mc = mappings.MappingConfig.build(model=self._model) if cfg is not None else None
    if mc is None or mc.to_hf_mappings is None:
      return list(params.items())
    plain = {n: p.detach() for n, p in params.items() if ".lora_" not in n}
    return list(mappings.apply(mc, plain).items())

  def update_params(self, params: Dict[str, torch.Tensor], filter_types: Optional[Tuple[Any, ...]] = None) -> None:
    del filter_types
    weights = self.hf_named_weights(params)
    if self._step_driver is not None:          # no engine step while the weights change
      self._step_driver.pause()
      try:
        self._push(weights)
      finally:
        self._step_driver.resume()
    else:
      self._push(weights)

  def _push(self, weights) -> None:
    loader = getattr(self.llm, "load_weights", None)
    if callable(loader):                     # injected engines and thin wrappers
      loader(weights)
      return
    # in-process engine: run the model's own `load_weights` on the (name, tensor) stream inside every worker. The
    # closure holds device tensors, so the engine core must live in this process (see `_in_process_engine`).
    apply = getattr(self.llm, "apply_model", None)
    if callable(apply):
      apply(lambda module: module.load_weights(iter(weights)) and None)
    else:
      self.llm.llm_engine.model_executor.driver_worker.model_runner.model.load_weights(weights)
    reset = getattr(self.llm, "reset_prefix_cache", None)
    if callable(reset):
      reset()

  # -- generation ------------------------------------------------------------------------------
  def _sampling_params(self, max_tokens, temperature, top_p, top_k, seed, eos_tokens, return_logprobs):
    kw = dict(max_tokens=int(max_tokens), temperature=float(temperature or 0.0),
              top_p=float(top_p) if top_p is not None else 1.0, top_k=int(top_k) if top_k else -1, seed=seed,
              stop_token_ids=list(eos_tokens) if eos_tokens else [self.tokenizer.eos_id()],
              logprobs=0 if return_logprobs else None, detokenize=False, skip_special_tokens=True)
    kw.update(self.config.sampling_kwargs)
    try:
      import vllm
      return vllm.SamplingParams(**kw)
    except ImportError:
      return kw                                # injected engines take the plain dict

  def generate_ids(self, prompt_ids: Sequence[Sequence[int]], params: Any) -> List[Any]:
    """Engine outputs for token-id prompts, through whichever path this sampler runs: the step-level driver
    (server mode on an engine that can be stepped), the batching thread around `generate`, or a direct call."""
    ids = [list(t) for t in prompt_ids]
    if self._step_driver is not None:
      futures = self._step_driver.submit_requests([{"prompt_token_ids": t} for t in ids], params)
      return [f.result(timeout=self.config.request_timeout_s) for f in futures]
    if self._driver is not None:
      req = self._driver.submit(ids, params)
      req.done.wait()
      if req.error is not None:
        raise req.error
      return req.result
    return self.llm.generate([{"prompt_token_ids": t} for t in ids], params, use_tqdm=False)

  def __call__(self, input_strings, max_generation_steps, max_prompt_length=None, temperature=0.0, top_p=None,
               top_k=None, beam_size=None, seed=None, multi_sampling: int = 1, return_logits: bool = False,
               echo: bool = False, pad_output: bool = False, eos_tokens: Optional[Sequence[int]] = None,
               return_logprobs: bool = False, **kwargs) -> base_sampler.SamplerOutput:
    if beam_size:
      raise NotImplementedError("beam search is not available through vLLM")
    strings = [input_strings] if isinstance(input_strings, str) else list(input_strings)
    ids = [self.tokenize(s).tolist() for s in strings]
    P = int(max_prompt_length or max(len(t) for t in ids))
    ids = [t[-P:] for t in ids]
    params = self._sampling_params(max_generation_steps, temperature, top_p, top_k, seed, eos_tokens,
                                   return_logprobs)
    outs = self.generate_ids(ids, params)
    eos = set(eos_tokens) if eos_tokens else {self.tokenizer.eos_id()}
    tokens, logprobs = [], []
    for o in outs:
      c = o.outputs[0]
      t = list(c.token_ids)
      lp = None
      if return_logprobs and getattr(c, "logprobs", None):
        lp = [float(next(iter(step.values())).logprob if not hasattr(step.get(tid, None), "logprob")
                    else step[tid].logprob) for tid, step in zip(t, c.logprobs)]
      if t and t[-1] in eos:
        t = t[:-1]
        lp = lp[:-1] if lp is not None else None
      tokens.append(np.asarray(t, dtype=np.int64))
      logprobs.append(lp)
    pad = self.tokenizer.pad_id()
    padded = np.full((len(ids), P), pad, dtype=np.int64)
    for i, t in enumerate(ids):
      padded[i, P - len(t):] = t
    text = [self.tokenizer.decode(t.tolist()) for t in tokens]
    if echo:
      text = [s + t for s, t in zip(strings, text)]
    return base_sampler.SamplerOutput(text=text, logits=[], tokens=tokens, padded_prompt_tokens=padded,
                                      logprobs=logprobs if return_logprobs else None)

  def close(self) -> None:
    if self._step_driver is not None:
      self._step_driver.shutdown()
    if self._driver is not None:
      self._driver.close()
    if self._tmp is not None:
      self._tmp.cleanup()
