"""Runner for the reference arm of `bench.py`: drives the unmodified reference package through its own
public API (`create_dummy_model` -> `PeftTrainer.train`, tunix/models/dummy_model_creator.py:30-92,
tunix/sft/peft_trainer.py:898-1112) on the same model, batch, sequence length and step counts as the
framework's own arm. Nothing of this repository's models, kernels or engine is imported here.

The reference needs jax, flax, optax (and the packages they pull in) with a CUDA backend; where they do not
import, `probe()` says which one is missing and the caller prints the `unavailable` line. One process per GPU
(the launcher's RANK / LOCAL_RANK / WORLD_SIZE) is mapped onto `jax.distributed` with one local device each.
"""
from __future__ import annotations

import os
import sys
import time
from typing import Any, Dict, Iterator, Optional

import numpy as np

_REF_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")
NEEDED = ("jax", "flax", "optax", "tunix")


def probe() -> Optional[str]:
  """None if the reference and what it runs on import; otherwise one line naming the first failure."""
  if not os.path.isdir(os.path.join(_REF_DIR, "tunix")):
    return "reference is not installed under baseline/_ref"
  if _REF_DIR not in sys.path:
    sys.path.insert(0, _REF_DIR)
  for name in NEEDED:
    try:
      __import__(name)
    except Exception as e:          # noqa: BLE001 - any import failure closes the arm
      return f"reference does not import offline: {type(e).__name__}: {e}"
  try:
    import jax
    if not any(d.platform == "gpu" for d in jax.devices()):
      return "jax imports but has no CUDA backend on this box"
  except Exception as e:            # noqa: BLE001
    return f"jax cannot enumerate devices: {type(e).__name__}: {e}"
  return None


class _TimedBatches:
  """Synthetic token batches from host memory, with a clock that starts when the first timed batch is asked
  for. `PeftTrainer.train` pulls one micro-batch per inner step, so batch number `warmup * accum` is the
  boundary; the device is drained there (through `drain`) before the clock is read."""

  def __init__(self, make_input, rows: int, seq_len: int, vocab: int, accum: int, warmup: int, steps: int, drain):
    self._make_input = make_input
    rng = np.random.default_rng(1234 + int(os.environ.get("RANK", "0")))
    self._pool = [rng.integers(1, vocab, size=(rows, seq_len), dtype=np.int32) for _ in range(4)]
    self._mask = np.ones((rows, seq_len), dtype=np.int32)
    self._first_timed = warmup * accum
    self._total = (warmup + steps) * accum
    self._drain = drain
    self.t_start: Optional[float] = None
    self.bytes_per_batch = self._pool[0].nbytes + self._mask.nbytes

  def __iter__(self) -> Iterator[Any]:
    for i in range(self._total):
      if i == self._first_timed:
        self._drain()
        self.t_start = time.perf_counter()
      yield self._make_input(input_tokens=self._pool[i % len(self._pool)], input_mask=self._mask)


def run(*, n_gpus: int, steps: int, warmup: int, global_batch: int, seq_len: int, micro_batch_per_gpu: int,
        model_name: str = "llama3p1_8b", learning_rate: float = 1e-5) -> Dict[str, Any]:
  """Trains `warmup + steps` optimizer steps with the reference's trainer and returns the timing of the last
  `steps`. Raises on any failure; the caller turns that into the `unavailable` line."""
  rank = int(os.environ.get("RANK", "0"))
  world = int(os.environ.get("WORLD_SIZE", "1"))
  import jax
  if world > 1:
    port = int(os.environ.get("MASTER_PORT", "29500")) + 17
    jax.distributed.initialize(coordinator_address=f"127.0.0.1:{port}", num_processes=world, process_id=rank,
                               local_device_ids=[int(os.environ.get("LOCAL_RANK", rank))])
  import jax.numpy as jnp
  import optax
  from flax import nnx
  from tunix.models import dummy_model_creator
  from tunix.models.llama3 import model as llama_lib
  from tunix.sft import peft_trainer
  from tunix.sft import utils as sft_utils

  devices = np.array(jax.devices()[:n_gpus]).reshape(n_gpus, 1)
  mesh = jax.sharding.Mesh(devices, ("fsdp", "tp"))
  config = getattr(llama_lib.ModelConfig, model_name)()
  model = dummy_model_creator.create_dummy_model(llama_lib.Llama3, config, mesh=mesh, dtype=jnp.bfloat16)

  rows = micro_batch_per_gpu * n_gpus                      # one micro-batch, whole job
  accum = max(1, global_batch // rows)
  trainer = peft_trainer.PeftTrainer(
      model, optax.adamw(learning_rate),
      peft_trainer.TrainingConfig(eval_every_n_steps=10**9, max_steps=warmup + steps,
                                  gradient_accumulation_steps=accum, pbar_description=None))

  def model_inputs(x):
    pad = x.input_tokens != 0
    return {"input_tokens": x.input_tokens, "input_mask": x.input_mask,
            "positions": sft_utils.build_positions_from_mask(pad),
            "attention_mask": sft_utils.make_causal_attn_mask(pad)}

  trainer = trainer.with_gen_model_input_fn(model_inputs)

  def drain():
    jax.block_until_ready(nnx.state(trainer.model))

  local_rows = rows // max(1, jax.process_count())
  batches = _TimedBatches(peft_trainer.TrainingInput, local_rows, seq_len, config.vocab_size, accum, warmup, steps, drain)
  with mesh:
    trainer.train(batches)
  drain()
  elapsed = time.perf_counter() - (batches.t_start or time.perf_counter())
  trainer.close()
  if world > 1:                                            # the slowest process sets the job's time
    from jax.experimental import multihost_utils
    elapsed = float(np.max(multihost_utils.process_allgather(np.float64(elapsed))))
  tokens = global_batch * seq_len * steps
  return {"tokens_per_s": tokens / elapsed, "ms_per_step": 1e3 * elapsed / steps, "accum": accum, "rows": rows,
          "h2d_bytes_per_step": batches.bytes_per_batch * accum, "rank": rank}
