"""Dataclass configs for trainers, rollout engines and RL clusters.

Field names, defaults and validation follow tunix/common/configs.py:60-407 so that user
code written against the reference keeps working. Differences that come from the execution
model (one process per GPU over NCCL instead of a single-controller device mesh):
`role_to_mesh` values are `tunix_b200.dist.Mesh` objects (named axes over ranks), and
optimizers are `tunix_b200.optim.GradientTransformation` factories.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Tuple, Union

from .datatypes import Mode, Role


def _is_positive_integer(value: Optional[int], name: str) -> None:
  if value is not None and (not isinstance(value, int) or isinstance(value, bool) or value <= 0):
    raise ValueError(f"{name} must be a positive integer, got {value!r}.")


def _check_divisibility(small: int, big: int, small_name: str, big_name: str) -> None:
  if big % small != 0:
    raise ValueError(f"{big_name} must be a multiple of {small_name}.")


@dataclasses.dataclass(frozen=True)
class CacheConfig:
  """Geometry of the KV cache."""

  cache_size: int
  num_layers: int
  num_kv_heads: int
  head_dim: int


@dataclasses.dataclass
class RolloutConfig:
  """Sampling and engine knobs of a rollout worker."""

  max_tokens_to_generate: int = 64
  temperature: float = 0.9
  top_p: Optional[float] = 1.0
  top_k: Optional[int] = None
  seed: Any = None
  max_prompt_length: int = 64
  kv_cache_size: int = 1024
  data_type: Any = None
  eos_tokens: Optional[List[int]] = None
  rollout_mapping_config: Any = None
  tensor_parallel_size: int = -1
  data_parallel_size: int = -1
  expert_parallel_size: int = 1
  return_logprobs: bool = False

  # Native engine (continuous batching, paged KV) knobs.
  page_size: int = 128
  max_running_requests: Optional[int] = None

  # vLLM engine knobs (accepted for configuration compatibility).
  rollout_vllm_server_mode: bool = False
  rollout_vllm_server_mode_submission_threshold: int = 0
  rollout_vllm_server_mode_submission_timeout_s: float = 0.0
  rollout_vllm_model_version: str = ""
  rollout_vllm_lora_config: Optional[Dict[str, Any]] = None
  rollout_vllm_hbm_utilization: float = 0.2
  rollout_vllm_init_with_random_weights: bool = True
  rollout_vllm_tpu_backend_type: Optional[str] = None
  rollout_vllm_async_scheduling: bool = False
  rollout_vllm_logprobs_mode: str = "processed_logprobs"
  rollout_vllm_hf_config_path: Optional[str] = None
  rollout_vllm_additional_config: Optional[Dict[str, Any]] = None
  rollout_vllm_enable_dp_attention: bool = False
  rollout_vllm_delete_dst_buffers: bool = True
  rollout_vllm_max_num_batched_tokens: Optional[int] = None
  rollout_vllm_max_num_seqs: Optional[int] = None
  rollout_vllm_reshard_chunk_size: Optional[int] = None
  rollout_vllm_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)
  rollout_vllm_sampling_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)

  # sglang engine knobs (accepted for configuration compatibility).
  rollout_sglang_jax_model_version: str = ""
  rollout_sglang_jax_context_length: Optional[int] = None
  rollout_sglang_jax_mem_fraction_static: float = 0.2
  rollout_sglang_jax_init_with_random_weights: bool = True
  rollout_sglang_jax_disable_radix_cache: bool = True
  rollout_sglang_jax_enable_deterministic_sampling: bool = False
  rollout_sglang_jax_use_sort_for_toppk_minp: bool = True
  rollout_sglang_jax_enable_static_lora: bool = False
  rollout_sglang_jax_enable_single_process: bool = True
  rollout_sglang_jax_lora_target_modules: Optional[List[str]] = None
  rollout_sglang_jax_max_lora_rank: Optional[int] = None
  rollout_sglang_jax_lora_scaling: Optional[float] = None
  rollout_sglang_jax_precompile_bs_paddings: Optional[List[int]] = None
  rollout_sglang_jax_precompile_token_paddings: Optional[List[int]] = None
  rollout_sglang_jax_chunked_prefill_size: Optional[int] = -1
  rollout_sglang_jax_page_size: int = 128
  rollout_sglang_jax_load_format: str = "auto"
  rollout_sglang_jax_max_running_requests: Optional[int] = None
  rollout_sglang_jax_log_level: Optional[str] = "info"
  rollout_sglang_jax_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)


@dataclasses.dataclass(kw_only=True)
class TrainingConfig:
  """Configuration of `PeftTrainer` and its subclasses."""

  eval_every_n_steps: int
  max_steps: Optional[int] = None
  gradient_accumulation_steps: Optional[int] = None
  checkpoint_root_directory: Optional[str] = None
  checkpointing_options: Any = None
  metrics_logging_options: Any = None
  profiler_options: Any = None
  perf_metrics_options: Any = None
  data_sharding_axis: Tuple[str, ...] = ("fsdp",)
  max_inflight_computations: int = 2
  metrics_prefix: str = ""
  pbar_description: Optional[str] = "Training"
  # Sequence packing: token budget per packed row (the reference's field name is kept).
  max_seq_token_per_tpu: Optional[int] = None
  max_segments_per_packed_row: Optional[int] = None
  # Global gradient-norm clip applied before the optimizer (None = no clipping).
  max_grad_norm: Optional[float] = None

  def get_with_default(self, key: str, default: Any) -> Any:
    val = getattr(self, key)
    return default if val is None else val


@dataclasses.dataclass(kw_only=True)
class RLTrainingConfig(TrainingConfig):
  """RL training config: optimizers and the batch-size hierarchy
  (global = dataloader batch x G; mini = one optimizer update; micro = one fwd/bwd)."""

  actor_optimizer: Any
  critic_optimizer: Any = None
  mini_batch_size: Optional[int] = None
  train_micro_batch_size: Optional[int] = None
  rollout_micro_batch_size: Optional[int] = None
  compute_logps_micro_batch_size: Optional[int] = None
  compute_logps_chunk_size: int = 0

  def __post_init__(self):
    for name in ("mini_batch_size", "train_micro_batch_size", "rollout_micro_batch_size",
                 "compute_logps_micro_batch_size", "max_segments_per_packed_row"):
      _is_positive_integer(getattr(self, name, None), name)
    if self.gradient_accumulation_steps is not None:
      raise ValueError("For RL training, gradient_accumulation_steps should be None. It is automatically "
                       "derived from: `mini_batch_size // train_micro_batch_size`.")
    if self.train_micro_batch_size is not None:
      if self.mini_batch_size is None:
        raise ValueError("For RL training, `mini_batch_size` must be set when `train_micro_batch_size` is set.")
      _check_divisibility(self.train_micro_batch_size, self.mini_batch_size,
                          f"{self.train_micro_batch_size=}", f"{self.mini_batch_size=}")
      self.gradient_accumulation_steps = self.mini_batch_size // self.train_micro_batch_size


@dataclasses.dataclass(kw_only=True, frozen=True)
class ClusterConfig:
  """Which ranks host which role, which rollout engine to use, and the training/rollout configs."""

  role_to_mesh: Dict[Role, Any]
  role_to_logical_axis_rule: Optional[Dict[Role, Any]] = None
  rollout_engine: Union[str, type] = "vanilla"
  offload_to_cpu: bool = False
  training_config: RLTrainingConfig
  rollout_config: Union[Dict[Mode, RolloutConfig], RolloutConfig]
