"""`rl/utils.py`: argument checks, batch slicing and merging, the critic wrapper, host offload, un-padding, and the
streaming sequence packer (placement, features, boundaries, errors, independence from producer granularity)."""
import dataclasses

import numpy as np
import pytest
import torch

from tunix_b200.rl import common, utils as rl_utils
from tests.test_rl_grpo import toy_model


# ---- small helpers ----------------------------------------------------------------------------------
@pytest.mark.parametrize("ok", [1, 7, np.int32(3), None])
def test_positive_integer_accepts(ok):
  rl_utils.is_positive_integer(ok, "n")


@pytest.mark.parametrize("bad", [0, -2, True, 1.0, "3"])
def test_positive_integer_rejects_and_names_the_argument(bad):
  with pytest.raises(ValueError, match="mini_batch_size must be a positive integer"):
    rl_utils.is_positive_integer(bad, "mini_batch_size")


def test_divisibility_and_chunk_slices():
  rl_utils.check_divisibility(4, 12, "micro", "mini")
  with pytest.raises(ValueError, match="mini must be a multiple of micro"):
    rl_utils.check_divisibility(5, 12, "micro", "mini")
  assert list(rl_utils.chunk_slices_by_size(7, 3)) == [slice(0, 3), slice(3, 6), slice(6, 7)]
  assert list(rl_utils.chunk_slices_by_size(0, 3)) == []


def test_weight_sharing_predicates():
  a = toy_model()
  b = toy_model()
  assert rl_utils.is_sharing_weights(a, a) and not rl_utils.is_sharing_weights(a, b)
  assert not rl_utils.is_sharing_weights(a, None) and not rl_utils.is_sharing_weights(None, None)
  from tunix_b200.models import lora as lora_lib
  import copy
  twin = copy.copy(a)                                   # same parameter objects under another module shell
  assert rl_utils.is_sharing_weights(a, twin)
  with_adapters = toy_model()
  for (_, p), (_, q) in zip(with_adapters.named_parameters(), a.named_parameters()):
    p.data = q.data                                     # backbone storage shared ...
  lora_lib.apply_lora_to_model(with_adapters, rank=2, alpha=4.0)      # ... adapters are its own
  assert rl_utils.is_sharing_backbone(a, with_adapters) and not rl_utils.is_sharing_weights(a, with_adapters)


def test_batch_slice_walks_dicts_lists_and_dataclasses():
  @dataclasses.dataclass
  class Ex:
    ids: torch.Tensor
    note: str
    extra: dict
  tree = {"a": np.arange(10).reshape(5, 2), "names": list("abcde"), "scalar": np.float32(3.0), "none": None,
          "ex": Ex(torch.arange(5), "keep", {"deep": torch.arange(10).view(5, 2)})}
  got = rl_utils.get_batch_slice(tree, slice(1, 3))
  assert got["a"].tolist() == [[2, 3], [4, 5]] and got["names"] == ["b", "c"] and got["scalar"] == 3.0
  assert got["none"] is None and got["ex"].ids.tolist() == [1, 2] and got["ex"].note == "keep"
  assert got["ex"].extra["deep"].tolist() == [[2, 3], [4, 5]]


def test_merge_micro_batches_by_kind():
  merged = rl_utils.merge_micro_batches([
      {"t": torch.tensor([1, 2]), "n": np.array([1.0]), "l": ["x"], "s": torch.tensor(5)},
      {"t": torch.tensor([3]), "n": np.array([2.0, 3.0]), "l": ["y", "z"], "s": torch.tensor(6)}])
  assert merged["t"].tolist() == [1, 2, 3] and merged["n"].tolist() == [1.0, 2.0, 3.0]
  assert merged["l"] == ["x", "y", "z"] and merged["s"].tolist() == [5, 6]
  assert rl_utils.merge_micro_batches([]) == {}


def test_critic_is_a_private_copy_with_a_scalar_head():
  actor = toy_model()
  critic = rl_utils.create_critic_model(actor, seed=3)
  assert not rl_utils.is_sharing_weights(actor, critic.transformer)
  tokens = torch.randint(3, 64, (2, 6), generator=torch.Generator().manual_seed(0))
  values, cache = critic(tokens)
  assert values.shape == (2, 6, 1) and cache is None
  hidden, _ = critic.transformer(tokens, skip_lm_head=True)
  torch.testing.assert_close(values[..., 0], hidden @ critic.score.w[0])
  again = rl_utils.create_critic_model(actor, seed=3)
  assert torch.equal(again.score.w, critic.score.w) and not torch.equal(
      rl_utils.create_critic_model(actor, seed=4).score.w, critic.score.w)
  with pytest.raises(ValueError, match="embed dim"):
    rl_utils.TransformerWithScoreHead(torch.nn.Linear(2, 2))


def test_offload_round_trip_keeps_values():
  m = toy_model()
  before = {n: p.detach().clone() for n, p in m.named_parameters()}
  rl_utils.put_params_on_memory_kind(m, "pinned_host")
  assert all(p.device.type == "cpu" for p in m.parameters())
  rl_utils.put_params_on_memory_kind(m, "device")
  for n, p in m.named_parameters():
    assert torch.equal(p.detach().cpu(), before[n])
  with pytest.raises(ValueError):
    rl_utils.put_params_on_memory_kind(m, "tape")


# ---- un-padding and packing -------------------------------------------------------------------------
def example(prompts, completions, advantages, P=4, C=5, with_logps=True, per_token_adv=False):
  """A padded TrainExample: prompts left-padded to P, completions right-padded to C; token values encode
  (sequence number, position) so that placement can be checked."""
  n = len(prompts)
  p_ids, p_mask = np.zeros((n, P), np.int64), np.zeros((n, P), np.int32)
  c_ids, c_mask = np.zeros((n, C), np.int64), np.zeros((n, C), np.int32)
  old = np.zeros((n, C), np.float32)
  for i, (p, c) in enumerate(zip(prompts, completions)):
    p_ids[i, P - len(p):], p_mask[i, P - len(p):] = p, 1
    c_ids[i, :len(c)], c_mask[i, :len(c)] = c, 1
    old[i, :len(c)] = [-0.1 * t for t in c]
  adv = np.asarray(advantages, np.float32)
  if per_token_adv:
    adv = np.repeat(adv[:, None], C, axis=1) * c_mask
  return common.TrainExample(prompt_ids=torch.as_tensor(p_ids), prompt_mask=torch.as_tensor(p_mask),
                             completion_ids=torch.as_tensor(c_ids), completion_mask=torch.as_tensor(c_mask),
                             advantages=torch.as_tensor(adv), ref_per_token_logps=None,
                             old_per_token_logps=torch.as_tensor(old) if with_logps else None)


def test_unpad_strips_both_sides_and_keeps_optional_fields_optional():
  ex = example([[11, 12], [21]], [[13, 14, 15], [22]], [0.5, -1.0])
  items = rl_utils.unpad_train_example(ex)
  assert [it["prompt_ids"].tolist() for it in items] == [[11, 12], [21]]
  assert [it["completion_ids"].tolist() for it in items] == [[13, 14, 15], [22]]
  assert items[0]["old_per_token_logps"].tolist() == pytest.approx([-1.3, -1.4, -1.5])
  assert items[0]["ref_per_token_logps"] is None and not items[0]["adv_is_per_token"] and float(items[1]["advantages"]) == -1.0
  bare = rl_utils.unpad_train_example(example([[1]], [[2, 3]], [1.0], with_logps=False))[0]
  assert bare["old_per_token_logps"] is None
  per_tok = rl_utils.unpad_train_example(example([[1]], [[2, 3]], [2.0], per_token_adv=True))[0]
  assert per_tok["adv_is_per_token"] and per_tok["advantages"].tolist() == [2.0, 2.0]


def _pack(stream, **kw):
  return [chunk[0] for chunk in rl_utils.pack_sequences(iter(stream), **kw)]


def test_packed_rows_hold_whole_sequences_with_their_features():
  ex = example([[11, 12], [21], [31, 32, 33]], [[13, 14], [22, 23, 24], [34]], [1.0, 2.0, 3.0])
  out = _pack([[ex]], max_token_budget=12, sequences_per_update=3, pack_size=1)
  assert len(out) == 1 and bool(out[0].is_update_step[0])
  row = out[0]
  ids, seg, pos = row.completion_ids[0].tolist(), row.segment_ids[0].tolist(), row.segment_positions[0].tolist()
  # first-fit decreasing: the two 4-token sequences first (input order among equals), then the other 4-token one
  sequences = {1: [11, 12, 13, 14], 2: [21, 22, 23, 24], 3: [31, 32, 33, 34]}
  placed = [tuple(ids[i] for i in range(12) if seg[i] == s) for s in (1, 2, 3)]
  assert sorted(placed) == sorted(tuple(v) for v in sequences.values()) and seg.count(0) == 0
  for s in (1, 2, 3):
    where = [i for i in range(12) if seg[i] == s]
    assert where == list(range(where[0], where[0] + 4)) and [pos[i] for i in where] == [0, 1, 2, 3]
  # the loss mask, advantages and old log-probs sit on completion tokens only and follow their tokens
  mask, adv, old = row.completion_mask[0].tolist(), row.advantages[0].tolist(), row.old_per_token_logps[0].tolist()
  for i, tok in enumerate(ids):
    is_completion = tok % 10 > {1: 2, 2: 1, 3: 3}[tok // 10]
    assert mask[i] == int(is_completion)
    assert adv[i] == (float(tok // 10) if is_completion else 0.0)
    assert old[i] == pytest.approx(-0.1 * tok if is_completion else 0.0)
  assert row.prompt_ids.shape == (1, 0) and row.num_segments == 13 and row.ref_per_token_logps is None


def test_token_only_stream_produces_no_logps_and_padding_is_segment_zero():
  ex = example([[11]], [[12, 13]], [1.0], with_logps=False)
  out = _pack([[ex]], max_token_budget=8, sequences_per_update=1, pad_id=99)
  assert out[0].old_per_token_logps is None
  assert out[0].completion_ids[0].tolist() == [11, 12, 13, 99, 99, 99, 99, 99]
  assert out[0].segment_ids[0].tolist() == [1, 1, 1, 0, 0, 0, 0, 0] and out[0].completion_mask[0].tolist() == [0, 1, 1, 0, 0, 0, 0, 0]


def test_several_rows_per_chunk_and_segment_cap():
  ex = example([[1]] * 6, [[2]] * 6, [1.0] * 6)
  two_rows = _pack([[ex]], max_token_budget=6, sequences_per_update=6, pack_size=2)
  assert len(two_rows) == 1 and two_rows[0].completion_ids.shape == (2, 6)
  assert sorted(int(r.max()) for r in two_rows[0].segment_ids) == [3, 3]
  capped = _pack([[ex]], max_token_budget=12, sequences_per_update=6, pack_size=1, max_segments_per_packed_row=2)
  assert len(capped) == 3 and all(int(c.segment_ids.max()) == 2 for c in capped) and capped[0].num_segments == 3
  assert [bool(c.is_update_step[0]) for c in capped] == [False, False, True]


def test_packing_does_not_depend_on_how_the_producer_batches():
  seqs = [([10 * k + 1], [10 * k + 2] * (1 + k % 3)) for k in range(1, 9)]
  def stream(group):
    return [[example([p for p, _ in seqs[i:i + group]], [c for _, c in seqs[i:i + group]], [1.0] * len(seqs[i:i + group]))]
            for i in range(0, 8, group)]
  def content(chunks):
    return sorted(tuple(t for t, s in zip(c.completion_ids[r].tolist(), c.segment_ids[r].tolist()) if s == k)
                  for c in chunks for r in range(c.completion_ids.shape[0]) for k in range(1, int(c.segment_ids[r].max()) + 1))
  a = _pack(stream(8), max_token_budget=8, sequences_per_update=8)
  b = _pack(stream(2), max_token_budget=8, sequences_per_update=8)
  assert content(a) == content(b) == sorted(tuple(p + c) for p, c in seqs)
  assert sum(bool(c.is_update_step[0]) for c in b) == 1 and bool(b[-1].is_update_step[0])


def test_chunks_stream_out_before_the_mini_batch_ends():
  """With more buffered tokens than a chunk holds, full chunks leave at once; the update flag waits for the end."""
  first = example([[1, 1]] * 4, [[2, 2]] * 4, [1.0] * 4)         # 16 tokens, budget 8
  second = example([[3]] * 2, [[4]] * 2, [1.0] * 2)
  produced = []
  gen = rl_utils.pack_sequences(iter([[first], [second]]), max_token_budget=8, sequences_per_update=6)
  produced.append(next(gen)[0])                                    # available after the first input alone
  assert not bool(produced[0].is_update_step[0])
  produced += [c[0] for c in gen]
  assert [bool(c.is_update_step[0]) for c in produced][-1] and sum(bool(c.is_update_step[0]) for c in produced) == 1
  assert sum(int((c.segment_ids > 0).sum()) for c in produced) == 16 + 4


def test_packer_errors():
  ok = example([[1]], [[2]], [1.0])
  with pytest.raises(ValueError, match="exceeding max_token_budget"):
    _pack([[example([[1, 1, 1, 1]], [[2, 2, 2, 2, 2]], [1.0])]], max_token_budget=8, sequences_per_update=1)
  with pytest.raises(ValueError, match="ended mid-mini-batch"):
    _pack([[ok]], max_token_budget=8, sequences_per_update=2)
  with pytest.raises(ValueError, match="boundary falls inside"):
    _pack([[example([[1]] * 3, [[2]] * 3, [1.0] * 3)]], max_token_budget=8, sequences_per_update=2)
  with pytest.raises(TypeError):
    rl_utils.pack_sequences(iter([[ok]]), max_token_budget=8)                  # sequences_per_update is required
  rl_utils.validate_packing_budget(16, 6, 10)
  with pytest.raises(ValueError, match="longest possible sequence"):
    rl_utils.validate_packing_budget(15, 6, 10)


def test_pack_size_follows_the_batch_axes():
  class Mesh:
    def __init__(self, **axes): self.axes = axes
    def axis_size(self, name): return self.axes.get(name, 1)
  assert rl_utils.compute_pack_size(None) == 1
  assert rl_utils.compute_pack_size(Mesh(fsdp=4, tp=2)) == 4 and rl_utils.compute_pack_size(Mesh(fsdp=2, dp=3)) == 6
