"""Shared machinery of the RL entry points (tunix/cli/base_rl_pipeline.py:47-902): role -> mesh
allocation with `same_mesh_as`, rollout / cluster / training configs, model creation (the
reference model is loaded once; the actor is its LoRA-wrapped or copied twin), critic score
head, dataset and step-count computation."""
from __future__ import annotations

import abc
import copy
import dataclasses
import importlib
import logging
from typing import Any, Dict, List, Mapping, MutableMapping, Optional, Tuple

import numpy as np
import torch

from ..common.configs import ClusterConfig, RLTrainingConfig, RolloutConfig
from ..common.datatypes import Mode, Role
from ..dist import mesh as dist_mesh
from ..perf import metrics as perf_metrics
from ..rl import rl_cluster as rl_engine_lib, utils as rl_utils
from ..utils import mesh as mesh_lib
from . import config
from .utils import data as data_lib, model as model_lib


class BasePipeline(abc.ABC, config.HyperParameters):
  _ROLE_TO_MODEL_KEY = {Role.ACTOR: "actor_model_config", Role.CRITIC: "critic_model_config",
                        Role.REFERENCE: "reference_model_config", Role.REWARD: "reward_model_config",
                        Role.ROLLOUT: "rollout_model_config"}
  _ROLE_ALIASES = {r.value.lower(): r for r in Role}

  def __init__(self, argv: List[str], **kwargs):
    super().__init__(argv, **kwargs)
    self.data_module = None

  @abc.abstractmethod
  def _default_training_mode(self) -> str: ...

  @abc.abstractmethod
  def _run(self, mode: str): ...

  def training_mode(self) -> str:
    return self.config.get("training_mode") or self._default_training_mode()

  @staticmethod
  def _is_agentic_mode(mode: str) -> bool:
    return mode.startswith("agentic")

  # ---- meshes --------------------------------------------------------------------------------
  def _resolve_split_role(self, name: str) -> Role:
    key = name.strip().lower()
    if key not in self._ROLE_ALIASES:
      raise ValueError(f"Unknown role name {name!r}. Expected one of {sorted(self._ROLE_ALIASES)}.")
    return self._ROLE_ALIASES[key]

  def _role_cfg(self, role: Role) -> Mapping[str, Any]:
    c = self.config.get(self._ROLE_TO_MODEL_KEY[role])
    return c if isinstance(c, Mapping) else {}

  def _is_role_active(self, role: Role) -> bool:
    if role in (Role.ACTOR, Role.REFERENCE, Role.ROLLOUT):
      return True
    return bool(self.config.get(self._ROLE_TO_MODEL_KEY[role]))

  def _get_same_mesh_as_map(self) -> Dict[Role, Role]:
    out = {}
    for role in self._ROLE_TO_MODEL_KEY:
      target = self._role_cfg(role).get("same_mesh_as")
      if target is None:
        continue
      if not isinstance(target, str):
        raise TypeError(f"Expected {self._ROLE_TO_MODEL_KEY[role]}.same_mesh_as to be None or str but got "
                        f"{type(target).__name__}")
      if role == Role.ACTOR:
        raise ValueError("Actor must own its mesh.")
      out[role] = self._resolve_split_role(target)
    return out

  def _resolve_mesh_owners(self) -> Dict[Role, Role]:
    """role -> the role whose mesh it uses: itself when it has a `mesh` section, the target of
    `same_mesh_as` (followed transitively), else the actor."""
    same = self._get_same_mesh_as_map()
    base: Dict[Role, Role] = {}
    for role in self._ROLE_TO_MODEL_KEY:
      if not self._is_role_active(role) and role not in same:
        continue
      base[role] = role if self._role_cfg(role).get("mesh") else Role.ACTOR
      if role in same and self._role_cfg(role).get("mesh"):
        raise ValueError(f"{self._ROLE_TO_MODEL_KEY[role]}.mesh is specified, so it must own a separate mesh and "
                         "cannot also use same_mesh_as.")

    def owner(role: Role, seen: set) -> Role:
      if role in seen:
        raise ValueError("same_mesh_as contains a cycle.")
      if role not in same:
        return base[role]
      seen.add(role)
      if same[role] not in base:
        raise ValueError(f"Role {same[role].value!r} is not active in this config.")
      return owner(same[role], seen)
    return {role: owner(role, set()) for role in base}

  def create_role_to_mesh(self) -> Dict[Role, Any]:
    """Every owner gets a disjoint slice of the job's ranks when the job has enough of them; a
    smaller job (one process, or fewer ranks than the owners ask for in total) colocates all
    owners on the same leading ranks, which is the single-node default of this platform."""
    role_to_owner = self._resolve_mesh_owners()
    owners: List[Role] = []
    for role in self._ROLE_TO_MODEL_KEY:
      if role in role_to_owner and role_to_owner[role] not in owners:
        owners.append(role_to_owner[role])
    policy = None
    reqs = []
    for o in owners:
      key = self._ROLE_TO_MODEL_KEY[o]
      shape, _ = self.parse_mesh_config(key)
      p = self._parse_mesh_allocation_policy(key)
      if policy is not None and p != policy:
        raise ValueError(f"All owned meshes must use the same mesh.allocation_policy, got {policy!r} and {p!r}.")
      policy = p
      reqs.append((key, int(np.prod(shape))))
    world = dist_mesh.world_size()
    if sum(n for _, n in reqs) <= world:
      slices = mesh_lib.allocate_named_mesh_device_slices(reqs, list(range(world)), policy or mesh_lib.COMPACT)
    else:
      too_big = [k for k, n in reqs if n > world]
      if too_big:
        raise ValueError(f"mesh of {too_big} needs more ranks than the job has ({world})")
      logging.info("roles ask for %d ranks in total but the job has %d: colocating them", sum(n for _, n in reqs), world)
      slices = {k: list(range(n)) for k, n in reqs}
    owner_mesh = {}
    for o in owners:
      key = self._ROLE_TO_MODEL_KEY[o]
      shape, names = self.parse_mesh_config(key)
      owner_mesh[o] = mesh_lib.create_mesh(shape, names, devices=slices[key])
    return {role: owner_mesh[o] for role, o in role_to_owner.items()}

  # ---- configs -------------------------------------------------------------------------------
  def _rollout_engine_extra(self, engine: str, kv_cache_size: int, max_running_requests: int,
                            role_to_mesh=None) -> Dict[str, Any]:
    extra: Dict[str, Any] = {}
    mesh = (role_to_mesh or {}).get(Role.ROLLOUT)
    if mesh is not None and "tp" in getattr(mesh, "axis_names", ()):
      extra["tensor_parallel_size"] = mesh.axis_size("tp")
    section = {"vllm": "vllm_config", "sglang_jax": "sglang_jax_config"}.get(engine)
    prefix = {"vllm": "rollout_vllm_", "sglang_jax": "rollout_sglang_jax_"}.get(engine, "")
    for k, v in (self.config.get(section) or {}).items() if section else []:
      extra[k if k.startswith(prefix) else prefix + k] = v
    if engine == "vllm":
      extra.setdefault("rollout_vllm_max_num_seqs", max_running_requests)
      if kv_cache_size:
        extra.setdefault("rollout_vllm_max_model_len", kv_cache_size)
    return extra

  def create_rollout_config(self, role_to_mesh=None) -> RolloutConfig:
    rc = self.config.get("rollout_config") or {}
    mode = self.training_mode()
    valid = {f.name for f in dataclasses.fields(RolloutConfig)}
    out = {k: v for k, v in rc.items() if k in valid}
    if "total_generation_steps" in rc:
      out["max_tokens_to_generate"] = rc["total_generation_steps"]
    p, g = rc.get("max_prompt_length", 0), rc.get("total_generation_steps", 0)
    algo = self.config.get(f"{mode}_config") or {}
    kv = 0
    if self._is_agentic_mode(mode) or (p and g):
      kv = p + g + 256
      out["kv_cache_size"] = kv
    if self._is_agentic_mode(mode):
      running = algo.get("max_concurrency", 16)
      out["return_logprobs"] = True
    else:
      running = self.config.get("batch_size", 1) * algo.get("num_generations", 1)
    extra = self._rollout_engine_extra(self.config.get("rollout_engine", "vanilla"), kv, running, role_to_mesh)
    out.update({k: v for k, v in extra.items() if k in valid})
    return RolloutConfig(**out)

  def create_rl_training_config(self) -> RLTrainingConfig:
    d = self.obtain_training_config_dict("rl_training_config")
    d["actor_optimizer"] = self.create_optimizer("rl_training_config", "actor_optimizer_config")
    if (self.config["rl_training_config"] or {}).get("critic_optimizer_config"):
      d["critic_optimizer"] = self.create_optimizer("rl_training_config", "critic_optimizer_config")
    return RLTrainingConfig(**d)

  def create_cluster_config(self, role_to_mesh, rollout_config) -> ClusterConfig:
    return ClusterConfig(role_to_mesh=role_to_mesh, rollout_engine=self.config.get("rollout_engine", "vanilla"),
                         offload_to_cpu=bool(self.config.get("offload_to_cpu", False)),
                         training_config=self.create_rl_training_config(), rollout_config=rollout_config)

  def create_perf_config(self, cluster_config: ClusterConfig):
    opts = cluster_config.training_config.perf_metrics_options
    if not opts:
      return None
    pc = perf_metrics.PerfMetricsConfig() if hasattr(perf_metrics, "PerfMetricsConfig") else None
    if pc is None:
      return opts
    if opts.custom_export_fn_path:
      pc.custom_export_fn = self._get_function_from_path(opts.custom_export_fn_path)
    if opts.custom_export_fn_path_v2:
      pc.custom_export_fn_v2 = self._get_function_from_path(opts.custom_export_fn_path_v2)
    return pc

  # ---- models --------------------------------------------------------------------------------
  def create_rl_engine(self, tokenizer):
    role_to_mesh = self.create_role_to_mesh()
    rollout_config = self.create_rollout_config(role_to_mesh)
    ref_cfg = dict(self.config["reference_model_config"])
    actor_cfg = dict(self.config["actor_model_config"])
    tok_cfg = self.config["tokenizer_config"]
    if ref_cfg.get("lora_config"):
      logging.warning("LoRA config is not supported for the reference model. Disabling LoRA.")
      ref_cfg.pop("lora_config")
    reference, _ = model_lib.create_model(ref_cfg, tok_cfg, role_to_mesh[Role.REFERENCE])
    if actor_cfg.get("lora_config"):
      # adapters on the shared frozen backbone: actor and reference use one set of base weights
      actor = model_lib.apply_lora_to_model(reference, role_to_mesh[Role.ACTOR], actor_cfg["lora_config"],
                                            rng_seed=actor_cfg.get("rng_seed", 0))
    else:
      actor = copy.deepcopy(reference)
      dt = actor_cfg.get("load_dtype")
      if dt:
        if not hasattr(torch, dt):
          raise ValueError(f"Invalid load_dtype: {dt}. Must be a valid torch dtype name.")
        actor = actor.to(getattr(torch, dt))
    critic = None
    critic_cfg = self.config.get("critic_model_config")
    if critic_cfg:
      critic, _ = model_lib.create_model(dict(critic_cfg), tok_cfg, role_to_mesh[Role.CRITIC])
      if hasattr(critic, "lm_head") or getattr(critic.config, "weight_tying", False):
        critic = rl_utils.create_critic_model(critic, seed=critic_cfg.get("rng_seed", 0))
      else:
        raise ValueError(f"Cannot create score head for Transformer backbone {critic_cfg.get('model_name')}.")
    cluster_config = self.create_cluster_config(role_to_mesh, rollout_config)
    kw = {}
    perf = self.create_perf_config(cluster_config)
    if perf is not None:
      kw["perf_config"] = perf
    return rl_engine_lib.RLCluster(actor=actor, critic=critic, reference=reference, tokenizer=tokenizer,
                                   cluster_config=cluster_config, **kw)

  create_rl_cluster = create_rl_engine

  # ---- data ----------------------------------------------------------------------------------
  def _compute_max_steps(self, dataset) -> int:
    rl = self.config["rl_training_config"]
    max_steps = rl.get("max_steps")
    try:
      n = len(dataset)
    except TypeError:
      n = None
      if not max_steps:
        raise ValueError("max_steps must be specified since the dataset length cannot be determined.") from None
    bs = self.config.get("batch_size", 1)
    nb = self.config.get("num_batches")
    if not nb and not n:
      raise ValueError("num_batches is not specified and cannot be determined since the dataset length is unknown.")
    if not nb:
      nb = n // bs
    self.config["num_batches"] = nb
    epochs = self.config.get("num_train_epochs") or 1
    frac = self.config.get("train_fraction")
    if not frac or frac <= 0.0 or frac > 1.0:
      frac = 0.8
    allowed = int(nb * epochs * frac)
    if not max_steps:
      return allowed
    if max_steps > allowed:
      raise ValueError(f"Maximum allowed value for max_steps is {allowed}, but {max_steps} is specified.")
    return max_steps

  def _apply_optimizer_step_limits(self, rl: MutableMapping[str, Any], key: str, max_steps: int) -> None:
    opt = rl.get(key)
    if opt is None:
      return
    if not isinstance(opt, MutableMapping):
      raise ValueError(f"rl_training_config.{key} must be a dict.")
    if opt and not opt.get("decay_steps"):
      opt["decay_steps"] = max_steps
    if opt and not opt.get("warmup_steps"):
      opt["warmup_steps"] = int(self.config.get("warmup_steps", self.config.get("warmup_ratio", 0.1) * max_steps))

  def compute_params(self, dataset) -> None:
    rl = self.config["rl_training_config"]
    max_steps = self._compute_max_steps(dataset)
    rl["max_steps"] = max_steps
    self._apply_optimizer_step_limits(rl, "actor_optimizer_config", max_steps)
    self._apply_optimizer_step_limits(rl, "critic_optimizer_config", max_steps)

  def _get_tokenizer(self):
    mc = self.config.get("actor_model_config") or self.config.get("model_config")
    return model_lib.create_tokenizer(self.config["tokenizer_config"], self.config["tokenizer_config"]["tokenizer_path"],
                                      model_config=mc)

  def _load_raw_dataset(self, tokenizer):
    src = self.config.get("data_source", "local")
    templ = bool(self.config.get("apply_chat_template_to_dataset"))
    if self.config.get("data_module"):
      return data_lib.get_dataset_from_module(self.config["data_module"], tokenizer, templ)
    from ..examples.data import math_dataset
    name = "synthetic" if src == "synthetic" else self.config["dataset_name"]
    ds = math_dataset.create_dataset(name, data_dir=self.config.get("data_directory", ""), as_messages=templ)
    if templ:
      import functools
      ds = ds.map(functools.partial(data_lib.apply_chat_template, tokenizer=tokenizer))
    return ds

  def _get_dataset(self, tokenizer):
    ds = self._load_raw_dataset(tokenizer)
    self.compute_params(ds)
    rc = self.config.get("rollout_config") or {}
    return data_lib.post_init_dataset(ds, tokenizer, batch_size=self.config["batch_size"],
                                      num_batches=self.config.get("num_batches"),
                                      max_prompt_length=rc.get("max_prompt_length"),
                                      fraction=self.config.get("train_fraction", 1.0),
                                      num_epochs=self.config.get("num_train_epochs", 1),
                                      prompt_key=self.config.get("prompt_key", "prompts"))

  def _load_class_from_path(self, dotted: str):
    mod, name = dotted.rsplit(".", 1)
    return getattr(importlib.import_module(mod), name)

  def _create_chat_parser(self, tokenizer):
    path = self.config.get("chat_parser_class")
    if not path:
      return None
    return self._load_class_from_path(path)(tokenizer)

  def run_trainer(self):
    mode = self.training_mode()
    logging.info("running %s in mode %s", type(self).__name__, mode)
    return self._run(mode)
