"""The dense-cache `Sampler`: output shapes under echo / padding / logits / log-probs, prompt length bucketing and
truncation, equality of batched and single decoding, state replacement (full and LoRA-only) with its checks, the
sampling primitives, a single generation step, and the cache-size guard."""
import numpy as np
import pytest
import torch

from tunix_b200.common.configs import CacheConfig
from tunix_b200.generate import sampler as sampler_lib
from tunix_b200.models import lora as lora_lib
from tests.test_rl_grpo import ToyTokenizer, toy_model


def make(model=None, cache=48):
  model = model or toy_model()
  cfg = model.config
  return sampler_lib.Sampler(model, ToyTokenizer(), CacheConfig(cache_size=cache, num_layers=cfg.num_layers,
                                                               num_kv_heads=cfg.num_kv_heads, head_dim=cfg.head_dim))


PROMPTS = ["alpha beta gamma delta", "one two", "x"]


# ---- primitives -------------------------------------------------------------------------------------
def test_top_p_and_top_k_masks_restrict_the_support():
  logits = torch.log(torch.tensor([[0.5, 0.3, 0.15, 0.05]])).repeat(400, 1)
  g = torch.Generator().manual_seed(0)
  everything, _ = sampler_lib.sample_top_p(logits, g, 1.0, 1.0, None)
  assert set(everything.tolist()) == {0, 1, 2, 3}
  nucleus, _ = sampler_lib.sample_top_p(logits, g, 1.0, 0.6, None)        # 0.5 alone is below 0.6: the next one joins
  assert set(nucleus.tolist()) == {0, 1}
  top2, lp = sampler_lib.sample_top_p(logits, g, 1.0, 1.0, 2, return_logprobs=True)
  assert set(top2.tolist()) == {0, 1}
  # reported log-probs are those of the unrestricted distribution at the given temperature
  assert float(lp[top2 == 0][0]) == pytest.approx(np.log(0.5), abs=1e-5)
  cold, _ = sampler_lib.sample_top_p(logits, g, 0.05, 1.0, None)
  assert (cold == 0).float().mean() > 0.99
  best, lp = sampler_lib.sample_best(logits[:2], return_logprobs=True)
  assert best.tolist() == [0, 0] and float(lp[0]) == pytest.approx(np.log(0.5), abs=1e-5)
  a = sampler_lib._step_generator(3, 5, "cpu").initial_seed()
  assert a == sampler_lib._step_generator(3, 5, "cpu").initial_seed() != sampler_lib._step_generator(3, 6, "cpu").initial_seed()


# ---- output contract ----------------------------------------------------------------------------------
@pytest.mark.parametrize("echo", [False, True])
@pytest.mark.parametrize("pad_output", [False, True])
def test_output_shapes_with_echo_padding_logits_and_logprobs(echo, pad_output):
  s = make()
  out = s(PROMPTS, max_generation_steps=5, max_prompt_length=8, echo=echo, pad_output=pad_output, return_logits=True,
          return_logprobs=True, eos_tokens=[10_000])
  prompt_lens = [len(s.tokenize(p)) for p in PROMPTS]
  assert out.padded_prompt_tokens.shape == (3, 8)
  for i, n in enumerate(prompt_lens):
    assert (out.padded_prompt_tokens[i, :8 - n] == 0).all() and (out.padded_prompt_tokens[i, 8 - n:] != 0).all()
  if pad_output:
    width = 13 if echo else 5
    assert np.asarray(out.tokens).shape == (3, width) and out.logits.shape[:2] == (3, width)
    assert all(len(lp) == width for lp in out.logprobs)
  else:
    for i, n in enumerate(prompt_lens):
      want = (n if echo else 0) + 5
      assert len(out.tokens[i]) == want and out.logits[i].shape == (want, 64) and len(out.logprobs[i]) == want
  assert len(out.text) == 3 and all(isinstance(t, str) for t in out.text)
  if echo and not pad_output:
    assert out.tokens[1][:prompt_lens[1]].tolist() == s.tokenize(PROMPTS[1]).tolist()


def test_logprobs_and_logits_describe_the_sampled_tokens():
  s = make()
  out = s(PROMPTS[:2], max_generation_steps=4, return_logits=True, return_logprobs=True, temperature=0.0, eos_tokens=[10_000])
  for toks, logits, lps in zip(out.tokens, out.logits, out.logprobs):
    assert toks.tolist() == logits.argmax(-1).tolist()                                # greedy picks the arg-max
    want = torch.log_softmax(logits, -1).gather(-1, torch.as_tensor(toks)[:, None])[:, 0]
    assert lps == pytest.approx(want.tolist(), abs=1e-5)


def test_a_batch_decodes_like_its_rows_alone():
  s = make()
  together = s(PROMPTS, max_generation_steps=6, eos_tokens=[10_000])
  for i, p in enumerate(PROMPTS):
    alone = s(p, max_generation_steps=6, eos_tokens=[10_000])
    assert alone.tokens[0].tolist() == together.tokens[i].tolist(), p


def test_prompt_length_is_bucketed_and_long_prompts_keep_their_tail():
  s = make(cache=64)
  five = "a b c d e"                                         # BOS + 5 tokens = 6 -> next power of two
  assert s(five, max_generation_steps=2).padded_prompt_tokens.shape == (1, 8)
  assert s(five, max_generation_steps=2, max_prompt_length=4).padded_prompt_tokens.shape == (1, 8)   # too small: raised
  assert s(five, max_generation_steps=2, max_prompt_length=16).padded_prompt_tokens.shape == (1, 16)
  with pytest.raises(ValueError, match="cache size"):
    s(five, max_generation_steps=60)


def test_one_generation_step_needs_no_decode_call():
  model = toy_model()
  calls = []
  forward = model.forward

  def counting(tokens, *a, **k):
    calls.append(tokens.shape[1])
    return forward(tokens, *a, **k)
  model.forward = counting
  out = make(model)(PROMPTS[:2], max_generation_steps=1, eos_tokens=[10_000])
  assert [len(t) for t in out.tokens] == [1, 1] and len(calls) == 1            # the prefill alone


def test_eos_ends_a_row_and_later_slots_are_padding():
  s = make()
  free = s(PROMPTS[0], max_generation_steps=6, eos_tokens=[10_000]).tokens[0].tolist()
  stop_at = free[2]
  cut = s(PROMPTS[0], max_generation_steps=6, eos_tokens=[stop_at], pad_output=True, return_logprobs=True)
  first = free.index(stop_at)
  assert cut.tokens[0][:first].tolist() == free[:first] and (cut.tokens[0][first:] == 0).all()
  assert all(v == 0.0 for v in cut.logprobs[0][first + 1:])
  banned = s(PROMPTS[0], max_generation_steps=6, eos_tokens=[10_000], forbidden_tokens=free[:1]).tokens[0].tolist()
  assert free[0] not in banned


# ---- replacing the weights ----------------------------------------------------------------------------
def test_full_state_replacement_changes_the_output_and_is_checked():
  s = make()
  before = s(PROMPTS[0], max_generation_steps=6, eos_tokens=[10_000]).tokens[0].tolist()
  donor = toy_model(seed=5)
  s.transformer_state = dict(donor.named_parameters())
  after = s(PROMPTS[0], max_generation_steps=6, eos_tokens=[10_000]).tokens[0].tolist()
  assert after == make(donor)(PROMPTS[0], max_generation_steps=6, eos_tokens=[10_000]).tokens[0].tolist() != before
  state = dict(donor.named_parameters())
  name = next(iter(state))
  with pytest.raises(ValueError, match="must cover all parameters"):
    s.transformer_state = {k: v for k, v in state.items() if k != name}
  with pytest.raises(ValueError, match="shape mismatch"):
    s.transformer_state = {**state, name: state[name][:1]}
  with pytest.raises(ValueError, match="dtype mismatch"):
    s.transformer_state = {**state, name: state[name].double()}
  assert s.dtype == torch.float32 and s.device.type == "cpu"


def test_lora_only_state_replacement():
  torch.manual_seed(0)
  model = toy_model()
  lora_lib.apply_lora_to_model(model, rank=2, alpha=4.0)
  s = make(model)
  base = {n: p.detach().clone() for n, p in model.named_parameters()}
  adapters = {n: torch.full_like(p, 0.05) for n, p in model.named_parameters() if getattr(p, "is_lora", False)}
  s.transformer_state = adapters
  for n, p in model.named_parameters():
    assert torch.equal(p, adapters[n] if n in adapters else base[n]), n
  some = dict(list(adapters.items())[:1])
  with pytest.raises(ValueError, match="exactly the LoRA parameters"):
    s.transformer_state = some
