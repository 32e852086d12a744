"""Layered run configuration (tunix/cli/config.py:170-1137).

Order of precedence: base YAML (first positional argument) < `override_config_file=<yaml>` <
`key=value` / `a.b.c=value` command-line overrides < `T_<KEY>` environment variables, where an
override given both on the command line and in the environment is an error. Unknown top-level
keys are rejected. Values are parsed as YAML scalars/collections and then coerced to the type of
the schema entry they replace; dict overrides merge into the schema entry except for the
sections in `REPLACE_KEYS`, which replace it whole. The four role model configs inherit
`model_config` values that they did not change themselves.
"""
from __future__ import annotations

import ast
import collections
import copy
import importlib
import importlib.util
import inspect
import logging
import os
import pathlib
import shutil
from typing import Any, Callable, Dict, List, Mapping, Optional, Sequence, Tuple

import yaml

from .. import optim

_ENV_PREFIX = "T_"
REPLACE_KEYS = frozenset({"lora_config", "training_config", "optimizer_config", "profiler_options", "rl_training_config"})
ROLE_MODEL_KEYS = ("actor_model_config", "critic_model_config", "reference_model_config", "rollout_model_config")
SUPPORTED_ENTRY_POINTS = ("peft_main", "grpo_main", "ppo_main")


def yaml_key_to_env_key(s: str) -> str:
  return _ENV_PREFIX + s.upper()


def string_to_bool(s: str) -> bool:
  if s.lower() == "true":
    return True
  if s.lower() == "false":
    return False
  raise ValueError(f"Can't convert {s} to bool")


def get_project_root() -> pathlib.Path:
  return pathlib.Path(__file__).resolve().parent.parent.parent


def _parse_scalar(text: str) -> Any:
  try:
    return yaml.safe_load(text)
  except yaml.YAMLError:
    return text


def parse_overrides(args: Sequence[str]) -> Dict[str, Any]:
  """["a.b=1", "c={x: 2}"] -> {"a": {"b": 1}, "c": {"x": 2}}."""
  out: Dict[str, Any] = {}
  for arg in args:
    if "=" not in arg:
      raise ValueError(f"override {arg!r} is not of the form key=value")
    key, val = arg.split("=", 1)
    node = out
    parts = key.strip().split(".")
    for p in parts[:-1]:
      node = node.setdefault(p, {})
      if not isinstance(node, dict):
        raise ValueError(f"override {arg!r} descends into a non-mapping")
    node[parts[-1]] = _parse_scalar(val)
  return out


def _coerce(schema_value: Any, value: Any, key: str) -> Any:
  """Types `value` like `schema_value` where a lossless conversion exists."""
  if value is None or schema_value is None:
    return value
  try:
    return _coerce_inner(schema_value, value, key)
  except ValueError as e:
    if "cannot turn" in str(e):
      raise
    raise ValueError(f"For key '{key}', cannot turn {value!r} into {type(schema_value).__name__}: {e}") from e


def _coerce_inner(schema_value: Any, value: Any, key: str) -> Any:
  if isinstance(schema_value, bool):
    if isinstance(value, bool):
      return value
    if isinstance(value, str):
      return string_to_bool(value)
  elif isinstance(schema_value, int) and not isinstance(schema_value, bool):
    if isinstance(value, (int, float)) and not isinstance(value, bool) and float(value).is_integer():
      return int(value)
    if isinstance(value, str):
      return int(value)
  elif isinstance(schema_value, float):
    if isinstance(value, (int, float, str)) and not isinstance(value, bool):
      return float(value)
  elif isinstance(schema_value, str):
    return value if isinstance(value, str) else str(value)
  elif isinstance(schema_value, (dict, list)):
    if isinstance(value, str):
      value = _parse_scalar(value)
    if isinstance(value, type(schema_value)):
      return value
  if isinstance(value, type(schema_value)):
    return value
  raise ValueError(f"For key '{key}', cannot turn {value!r} ({type(value).__name__}) into "
                   f"{type(schema_value).__name__}")


def update_dict(schema: Mapping[str, Any], source: Mapping[str, Any], replace_keys=REPLACE_KEYS) -> Dict[str, Any]:
  out = copy.deepcopy(dict(schema))
  for k, v in source.items():
    if k not in replace_keys and isinstance(v, Mapping) and isinstance(out.get(k), Mapping):
      out[k] = update_dict(out[k], v, replace_keys)
    else:
      out[k] = copy.deepcopy(v) if k not in out or isinstance(v, Mapping) else _coerce(out[k], v, k)
  return out


def _flatten(d: Mapping[str, Any], prefix: str = "") -> List[str]:
  out = []
  for k, v in d.items():
    if isinstance(v, Mapping) and v and k not in REPLACE_KEYS:
      out += _flatten(v, f"{prefix}{k}.")
    else:
      out.append(f"{prefix}{k}={yaml.safe_dump(v, default_flow_style=True).strip().removesuffix('...').strip()}")
  return out


class HyperParameters:
  """`HyperParameters(argv)` with argv = [entry point, base yaml, overrides...]; the merged
  configuration is the plain dict `self.config`."""

  SUPPORTED_MODEL_SOURCES = ("kaggle", "huggingface", "gcs", "internal", "maxtext", "orbax", "dummy", "")

  def __init__(self, argv: List[str], **kwargs):
    if len(argv) < 2 or "=" in argv[1]:
      raise ValueError("The first argument must be a path to a base config file.")
    here = pathlib.Path(__file__).parent
    base_file = here / argv[1] if argv[1] in ("base_config.yaml", "base_agentic_config.yaml") else argv[1]
    schema = self._load_config_from_yaml(str(base_file))
    self._validate_env_variable(schema)
    base_model_config = copy.deepcopy(schema.get("model_config") or {})
    self.replace_keys = set(REPLACE_KEYS)
    file_override, cli = None, []
    for arg in argv[2:]:
      if arg.startswith("override_config_file="):
        if file_override is not None:
          raise ValueError("Only one override_config_file argument is allowed.")
        file_override = arg.split("=", 1)[1]
      else:
        cli.append(arg)
    overrides: Dict[str, Any] = {}
    if file_override:
      overrides = update_dict(overrides, self._load_config_from_yaml(file_override), frozenset())
    overrides = update_dict(overrides, parse_overrides(cli), frozenset())
    self.config: Dict[str, Any] = collections.OrderedDict()
    self._update_from_env_and_command_line(self.config, schema, overrides)
    model_cfg = self.config.get("model_config") or {}
    for key in ROLE_MODEL_KEYS:
      role = self.config.get(key)
      if role is not None:
        for k, v in model_cfg.items():
          if k not in role or role[k] == base_model_config.get(k):
            role[k] = copy.deepcopy(v)
    self._validate_tokenizer()
    self._validate_model_source(self.config)
    self.check_supported_workflow()
    self._validate_perf_metrics(entry_point=argv[0])

  # ---- loading and merging -------------------------------------------------------------------
  @staticmethod
  def _load_config_from_yaml(path: str) -> Dict[str, Any]:
    try:
      with open(path) as f:
        data = yaml.safe_load(f) or {}
    except FileNotFoundError as e:
      raise ValueError(f"Config {path} not found.") from e
    if not isinstance(data, dict):
      raise ValueError(f"Config {path} must be a mapping at the top level.")
    return data

  @staticmethod
  def _validate_env_variable(schema: Mapping[str, Any]) -> None:
    for name in os.environ:
      if name.startswith(_ENV_PREFIX):
        rest = name[len(_ENV_PREFIX):]
        if rest.lower() not in schema:
          raise ValueError(f"We received env {name} but it doesn't match a key, so it is assumed a mistake.")
        if not rest.isupper():
          raise ValueError(f"We received env {name} but it isn't all uppercase.")

  def _update_from_env_and_command_line(self, out: Dict[str, Any], schema: Mapping[str, Any],
                                        overrides: Mapping[str, Any]) -> List[str]:
    for k in overrides:
      if k and k not in schema:
        raise ValueError(f"Key {k} was passed at the command line but isn't in config.")
    changed = []
    for k, base in schema.items():
      env_key = yaml_key_to_env_key(k)
      in_cli, in_env = k in overrides, env_key in os.environ
      if in_cli and in_env:
        raise ValueError(f"You are passing overrides by both CLI and ENV for `{k}`. This isn't allowed.")
      if not in_cli and not in_env:
        out[k] = copy.deepcopy(base)
        continue
      changed.append(k)
      new = overrides[k] if in_cli else _parse_scalar(os.environ[env_key])
      if base is None:
        if new is not None and not isinstance(new, (dict, list, str, int, float, bool)):
          raise ValueError(f"For key '{k}', nullable schema can't accept value of type {type(new)} from the CLI or ENV")
        out[k] = copy.deepcopy(new)
      elif isinstance(base, Mapping):
        new = _coerce(base, new, k)
        out[k] = copy.deepcopy(new) if k in self.replace_keys else update_dict(base, new, self.replace_keys)
      else:
        out[k] = _coerce(base, new, k)
    return changed

  def update_dict(self, schema, source):
    return update_dict(schema, source, self.replace_keys)

  # ---- validation ----------------------------------------------------------------------------
  def _validate_tokenizer(self) -> None:
    tc = self.config.get("tokenizer_config") or {}
    ttype, path = tc.get("tokenizer_type"), tc.get("tokenizer_path", "")
    valid = {"sentencepiece", "huggingface"}
    if ttype not in valid:
      raise ValueError(f"tokenizer_type {ttype} is not supported, currently only {valid} is supported")
    if ttype == "huggingface":
      if not path:
        raise ValueError("tokenizer_path must be specified.")
      local = path.startswith(("/", ".", "gs://")) or os.path.exists(path)
      if not local and "HF_TOKEN" not in os.environ:
        raise ValueError("Missing `HF_TOKEN` to access hf tokenizer")

  def _validate_model_source(self, cfg: Mapping[str, Any]) -> None:
    mc = cfg.get("model_config") or {}
    src = mc.get("model_source")
    if src not in self.SUPPORTED_MODEL_SOURCES:
      raise ValueError(f"Invalid model_source: {src!r}. Must be one of {self.SUPPORTED_MODEL_SOURCES}.")
    if src in ("kaggle", "huggingface") and not mc.get("intermediate_ckpt_dir"):
      raise ValueError("intermediate_ckpt must be specified when model_source is 'kaggle' or 'huggingface'")

  def check_supported_workflow(self) -> None:
    mc = self.config["model_config"]
    name, src = mc["model_name"], mc["model_source"]
    table = {"gemma": ["kaggle", "internal", "maxtext"], "gemma2": ["kaggle", "internal", "maxtext"],
             "gemma3": ["gcs", "internal", "maxtext"], "gemma4": ["kaggle", "huggingface", "gcs", "internal"]}
    fam = "other"
    for prefix, f in (("gemma4", "gemma4"), ("gemma-4", "gemma4"), ("gemma3", "gemma3"), ("gemma-3", "gemma3"),
                      ("gemma2", "gemma2"), ("gemma-2", "gemma2"), ("gemma", "gemma")):
      if name.startswith(prefix):
        fam = f
        break
    # local safetensors / Orbax directories and random weights work for every family
    expected = table.get(fam, ["huggingface", "internal", "maxtext"]) + ["orbax", "dummy", "huggingface"]
    if src not in expected:
      raise ValueError(f"Model '{name}' must use source(s) {expected}, but got '{src}'.")

  def _validate_perf_metrics(self, entry_point: str) -> None:
    perf = (self.config.get("training_config") or {}).get("perf_metrics_options") or {}
    if not perf:
      return
    if not os.path.splitext(os.path.basename(entry_point))[0].endswith("grpo_main"):
      raise ValueError("Perf metrics are currently only supported for GRPO training (grpo_main).")
    for key, what in (("custom_export_fn_path", "custom export function"),
                      ("custom_export_fn_path_v2", "custom export function v2")):
      path = perf.get(key)
      if path and self._get_function_from_path(path) is None:
        raise ValueError(f"Could not load {what} from {path}")

  def clear_directory_contents(self) -> None:
    path = self.config.get("model_download_path") or self.config["model_config"].get("model_download_path")
    if not path or not os.path.isdir(path):
      logging.error("Error: '%r' is not a valid directory.", path)
      return
    for item in os.listdir(path):
      full = os.path.join(path, item)
      try:
        if os.path.isdir(full) and not os.path.islink(full):
          shutil.rmtree(full)
        else:
          os.remove(full)
      except OSError:
        logging.warning("  Failed to delete %s.", full, exc_info=True)

  # ---- factories -----------------------------------------------------------------------------
  def _get_nested_config(self, keys: Sequence[str]) -> Any:
    cur: Any = self.config
    for i, k in enumerate(keys):
      if not isinstance(cur, Mapping):
        raise TypeError(f"Attempted to access key '{k}' on a non-dictionary element at path: {' -> '.join(keys[:i])}")
      if k not in cur:
        raise KeyError(f"Key '{k}' not found in config path: {' -> '.join(keys[:i + 1])}")
      cur = cur[k]
    return cur

  @staticmethod
  def _extract_kwargs(func: Callable[..., Any], config: Mapping[str, Any], where: str,
                      learning_rate: Any = None) -> Dict[str, Any]:
    kw = {}
    for p in inspect.signature(func).parameters.values():
      if p.kind in (p.VAR_KEYWORD, p.VAR_POSITIONAL):
        continue
      if p.name in config and not (p.name == "learning_rate" and learning_rate is not None):
        kw[p.name] = config[p.name]
      elif learning_rate is not None and p.name == "learning_rate":
        kw[p.name] = learning_rate
      elif p.default is p.empty:
        raise ValueError(f"Missing required argument '{p.name}' for {getattr(func, '__name__', func)} in config at "
                         f"{where}.")
    return kw

  def _create_learning_rate(self, oc: Mapping[str, Any], where: str) -> Any:
    st = oc.get("schedule_type")
    if st:
      try:
        fn = optim.get_schedule_factory(st)
      except (KeyError, AttributeError, ValueError) as e:
        raise AttributeError(f"Config {where}: '{st}' is not a valid schedule.") from e
      return fn(**self._extract_kwargs(fn, oc, where))
    lr = oc.get("learning_rate")
    if lr is not None and not isinstance(lr, (int, float)):
      raise TypeError(f"learning_rate must be a scalar when no schedule_type is specified, got {type(lr)} in config "
                      f"at {where}.")
    return lr

  def create_optimizer(self, *optimizer_keys: str) -> optim.GradientTransformation:
    """Optimizer from e.g. ("rl_training_config", "actor_optimizer_config"): any optimizer of
    `tunix_b200.optim` by `opt_type`, any schedule by `schedule_type`, arguments picked from the
    section by signature, hyper-parameters readable at run time, optional `max_grad_norm` clip."""
    if not optimizer_keys:
      raise ValueError("At least one optimizer key must be provided.")
    where = " -> ".join(optimizer_keys)
    try:
      oc = self._get_nested_config(optimizer_keys)
    except KeyError as e:
      raise KeyError(f"Could not resolve optimizer config path: {e}") from e
    if not isinstance(oc, Mapping):
      raise ValueError("optimizer_config must be a dictionary")
    opt_type = oc.get("opt_type")
    if not opt_type:
      raise ValueError("Optimizer name is required")
    try:
      factory = optim.get_optimizer_factory(opt_type.lower())
    except (KeyError, AttributeError, ValueError) as e:
      raise ValueError(f"Optimizer type '{opt_type}' not supported from {where}.") from e
    lr = self._create_learning_rate(oc, where)
    params = inspect.signature(factory).parameters
    if lr is None and "learning_rate" in params and params["learning_rate"].default is inspect.Parameter.empty:
      raise ValueError(f"Missing required argument 'learning_rate' for optimizer '{opt_type}' and no schedule defined "
                       f"in config at {where}.")
    kw = self._extract_kwargs(factory, oc, where, lr)
    try:
      tx = optim.inject_hyperparams(factory)(**kw)
    except TypeError as e:
      raise TypeError(f"Error calling {opt_type} with arguments {kw}: {e}") from e
    clip = oc.get("max_grad_norm")
    return optim.chain(optim.clip_by_global_norm(float(clip)), tx) if clip else tx

  def parse_mesh_config(self, model_key: str) -> Tuple[Tuple[int, ...], Tuple[str, ...]]:
    mesh = (self.config.get(model_key) or {}).get("mesh")
    if not mesh:
      raise ValueError("Missing 'mesh' configuration in raw_keys.")
    if not isinstance(mesh, Mapping):
      raise ValueError(f"The 'mesh' configuration must be a dictionary-like object, got {type(mesh)}.")
    out = []
    for field in ("shape", "axis_names"):
      raw = mesh.get(field)
      if not raw:
        raise ValueError(f"Missing '{field}' key in 'mesh' configuration.")
      try:
        val = ast.literal_eval(raw) if isinstance(raw, str) else tuple(raw)
      except (ValueError, SyntaxError) as e:
        raise ValueError(f"Invalid '{field}' key in 'mesh' configuration: {raw}") from e
      if isinstance(val, list):
        val = tuple(val)
      if not isinstance(val, tuple):
        raise ValueError(f"'mesh.{field}' must be a tuple, got {type(val)}.")
      out.append(val)
    shape, names = out
    if not all(isinstance(x, int) and not isinstance(x, bool) for x in shape):
      raise ValueError(f"All elements in mesh.shape must be integers, got {shape}.")
    if not all(isinstance(x, str) for x in names):
      raise ValueError(f"All elements in mesh.axis_names must be strings, got {names}.")
    if len(shape) != len(names):
      raise ValueError(f"mesh.shape {shape} and mesh.axis_names {names} must have the same length.")
    return shape, names

  def _parse_mesh_allocation_policy(self, model_key: str) -> str:
    mesh = (self.config.get(model_key) or {}).get("mesh")
    if not mesh or not isinstance(mesh, Mapping):
      raise ValueError("Missing 'mesh' configuration in raw_keys.")
    from ..utils import mesh as mesh_lib
    return mesh_lib.normalize_allocation_policy(mesh.get("allocation_policy"))

  def obtain_training_config_dict(self, key: str) -> Dict[str, Any]:
    """The section `key` with its option sub-sections turned into their option objects."""
    from ..perf import metrics as perf_metrics
    from ..sft import checkpoint_options, metrics_logger, profiler
    tc = self.config[key]
    if not isinstance(tc, Mapping):
      raise ValueError(f"Expected 'training_config' to be a dictionary, but got {type(tc).__name__}")
    builders = {"checkpointing_options": checkpoint_options.checkpointing_options_from_dict,
                "metrics_logging_options": lambda v: metrics_logger.MetricsLoggerOptions(**v),
                "profiler_options": lambda v: profiler.ProfilerOptions(**v),
                "perf_metrics_options": lambda v: perf_metrics.PerfMetricsOptions(**v)}
    out: Dict[str, Any] = {}
    for k, v in tc.items():
      if "optimizer_config" in k:
        continue
      if k in builders:
        if not v:
          out[k] = None
          continue
        if not isinstance(v, Mapping):
          raise ValueError(f"Expected dictionary for {k}, but got {type(v).__name__}")
        try:
          out[k] = builders[k](v)
        except (ValueError, TypeError) as e:
          raise ValueError(f"Invalid {k.replace('_', ' ')}: {v}") from e
      else:
        out[k] = v
    return out

  # ---- reward functions ----------------------------------------------------------------------
  def _load_module(self, ref: str):
    if "/" not in ref and not ref.endswith(".py"):
      try:
        return importlib.import_module(ref)
      except Exception as e:
        logging.warning("'%s' import failed: %s", ref, e)
    path = ref if os.path.isabs(ref) else str(get_project_root() / ref)
    name = os.path.splitext(os.path.basename(path))[0]
    spec = importlib.util.spec_from_file_location(name, path)
    if spec is None or spec.loader is None:
      raise ImportError(f"Cannot find spec for module at {path}")
    mod = importlib.util.module_from_spec(spec)
    try:
      spec.loader.exec_module(mod)
    except Exception as e:
      raise ImportError(f"Failed to execute module {name} from {path}") from e
    return mod

  def obtain_reward_fn(self) -> List[Callable[..., Any]]:
    """Every public function defined in each listed module (path or dotted name); with
    `verl_compatible`, an adapter around the module's `compute_score(completion, ground_truth)`."""
    fns: List[Callable[..., Any]] = []
    for ref in self.config.get("reward_functions") or []:
      mod = self._load_module(ref)
      if self.config.get("verl_compatible"):
        def reward_fn(prompts, completions, reward_model, *, _m=mod, **kwargs):
          return [_m.compute_score(c, gt) for c, gt in zip(completions, reward_model["ground_truth"])]
        fns.append(reward_fn)
      else:
        fns += [m for n, m in inspect.getmembers(mod, inspect.isfunction)
                if not n.startswith("_") and m.__module__ == mod.__name__]
    return fns

  @staticmethod
  def _get_function_from_path(path_str: str):
    try:
      module_path, name = path_str.rsplit(".", 1)
      return getattr(importlib.import_module(module_path), name)
    except (ImportError, AttributeError, ValueError) as e:
      logging.warning("Error importing '%s': %s", path_str, e)
      return None


def initialize(argv: List[str], **kwargs) -> HyperParameters:
  return HyperParameters(argv, **kwargs)
