"""Dataset plumbing of the command-line entry points (tunix/cli/utils/data.py:27-261)."""
from __future__ import annotations

import ast
import dataclasses
import functools
import importlib
import importlib.util
import os
import re
from typing import Any, Callable, Dict, List, Optional, Tuple

from ...data import ListDataset
from ...utils import token_sanitization


def apply_chat_template(x: Dict[str, Any], tokenizer) -> Dict[str, Any]:
  """{"prompt": messages, ...} -> {"prompts": rendered text, ...}."""
  return {"prompts": tokenizer.apply_chat_template(x["prompt"], tokenize=False, add_generation_prompt=True),
          **{k: v for k, v in x.items() if k != "prompt"}}


def parse_call_string(arg_string: str) -> Tuple[List[Any], Dict[str, Any]]:
  """"'a', 1, k='v'" -> (['a', 1], {'k': 'v'}); literals only."""
  if not arg_string.strip():
    return [], {}
  try:
    tree = ast.parse(f"f({arg_string})", mode="eval")
  except SyntaxError as e:
    raise ValueError(f"Invalid argument syntax: {arg_string}") from e
  call = tree.body
  if not isinstance(call, ast.Call):
    raise ValueError(f"Internal error: Expected a Call node for '{arg_string}'")
  return [ast.literal_eval(a) for a in call.args], {k.arg: ast.literal_eval(k.value) for k in call.keywords}


def _load_module(where: str):
  """A dotted module name, or the path of a `.py` file (loaded under its base name)."""
  from_file = where.endswith(".py") and os.path.exists(where)
  try:
    if not from_file:
      return importlib.import_module(where)
    name = os.path.splitext(os.path.basename(where))[0]
    spec = importlib.util.spec_from_file_location(name, where)
    if spec is None or spec.loader is None:
      raise ImportError(f"Failed to create spec for {where}")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module
  except ImportError:
    raise
  except Exception as e:
    raise ImportError(f"Failed to import module {where}: {e}") from e


@dataclasses.dataclass(frozen=True)
class DatasetSpec:
  """`module[:function[(literal arguments)]]`; `module` may be a file path, also one with a drive letter."""
  module: str
  function: str = "create_dataset"
  args: Tuple[Any, ...] = ()
  kwargs: Tuple[Tuple[str, Any], ...] = ()

  _FORM = re.compile(r"^(?P<module>(?:[A-Za-z]:(?=[\\/]))?[^:]+)(?::(?P<function>[A-Za-z_]\w*)(?:\((?P<call>.*)\))?)?$", re.S)

  @classmethod
  def parse(cls, text: str) -> "DatasetSpec":
    m = cls._FORM.match(text.strip())
    if m is None:
      raise ValueError(f"cannot read dataset specifier {text!r}: expected module[:function[(arguments)]]")
    args, kwargs = parse_call_string(m["call"]) if m["call"] else ([], {})
    return cls(m["module"], m["function"] or "create_dataset", tuple(args), tuple(kwargs.items()))

  def build(self, **defaults):
    """Calls the function; arguments written in the specifier win over `defaults`."""
    return getattr(_load_module(self.module), self.function)(*self.args, **{**defaults, **dict(self.kwargs)})


def get_dataset_from_module(specifier: str, tokenizer=None, apply_chat_template_to_dataset: bool = False,
                            **dataset_kwargs):
  """`pkg.mod`, `pkg.mod:func`, `pkg.mod:func('x', split='train')` or `/path/file.py:func`;
  the default function is `create_dataset`."""
  ds = DatasetSpec.parse(specifier).build(**dataset_kwargs)
  if not apply_chat_template_to_dataset:
    return ds
  if tokenizer is None:
    raise ValueError("tokenizer must be provided when apply_chat_template_to_dataset is True.")
  as_mappable = ds if hasattr(ds, "map") else ListDataset(list(ds))
  return as_mappable.map(functools.partial(apply_chat_template, tokenizer=tokenizer))


def post_init_dataset(dataset, tokenizer, batch_size: int, num_batches: Optional[int], max_prompt_length: Optional[int],
                      fraction: float = 1.0, num_epochs: int = 1, prompt_key: str = "prompts",
                      custom_batch_fn: Optional[Callable] = None):
  """Filters over-long prompts, truncates to `num_batches`, splits by `fraction`, repeats and
  batches. Returns (first split, second split or None) as re-iterable batch streams."""
  if not hasattr(dataset, "map"):
    dataset = ListDataset(list(dataset))
  original = len(dataset)
  if prompt_key != "prompts":
    src = prompt_key
    dataset = dataset.map(lambda x: {**x, "prompts": token_sanitization.sanitize_control_tokens(x[src])})
    prompt_key = "prompts"
  if max_prompt_length is not None and max_prompt_length > 0:
    dataset = dataset.filter(lambda x: len(tokenizer.encode(x[prompt_key])) <= max_prompt_length)
  filtered = len(dataset)
  if filtered == 0:
    raise ValueError("Training dataset is empty after post_init_dataset filtering. "
                     f"original_size={original}, max_prompt_length={max_prompt_length}, prompt_key={prompt_key!r}. "
                     "Consider increasing max_prompt_length or adjusting the prompt template/filter settings.")
  if num_batches is not None and num_batches > 0:
    dataset = dataset[:min(num_batches * batch_size, len(dataset))]
  first, second = dataset, None
  if 0.0 < fraction < 1.0:
    cut = int(len(dataset) * fraction)
    first, second = dataset[:cut], dataset[cut:]
  if len(first) == 0:
    raise ValueError("Training dataset is empty after post_init_dataset split. "
                     f"filtered_size={filtered}, fraction={fraction}, num_batches={num_batches}, batch_size={batch_size}.")
  mk = lambda d: d.repeat(num_epochs).to_iter_dataset().batch(batch_size, batch_fn=custom_batch_fn)
  return mk(first), (mk(second) if second is not None else None)
