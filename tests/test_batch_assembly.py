"""Batch assemblers of the experimental plane: padding helpers, reference log-prob attachment, the GRPO assembler
(prompt / completion layout, truncation, optional fields, filler rows, chunking) and the two token-stream
assemblers (fixed rectangular batches and sequence packing)."""
import numpy as np
import pytest

from tunix_b200.experimental.common import datatypes
from tunix_b200.experimental.orchestrator import batch_assembly as ba
from tunix_b200.rl import common as rl_common


def payload(tokens, loss=None, adv=1.0, **kw):
  tokens = np.asarray(tokens, np.int32)
  loss = np.ones(len(tokens), np.float32) if loss is None else np.asarray(loss, np.float32)
  return datatypes.RLTrainerPayload(token_ids=tokens, token_mask=np.ones(len(tokens), np.float32), loss_mask=loss,
                                    advantages=adv, **kw)


def grpo_item(prompt, completion, adv=1.0, **kw):
  return payload(list(prompt) + list(completion), adv=adv, prompt_ids=np.asarray(prompt), completion_ids=np.asarray(completion),
                 **kw)


# ---- helpers ------------------------------------------------------------------------------------------
def test_padding_helpers():
  ids, mask = ba._left_pad(np.array([5, 6], np.int32), 4, 9)
  assert ids.tolist() == [9, 9, 5, 6] and mask.tolist() == [0, 0, 1, 1]
  ids, mask = ba._left_pad(np.array([1, 2, 3, 4, 5], np.int32), 3, 9)            # the tail survives
  assert ids.tolist() == [3, 4, 5] and mask.tolist() == [1, 1, 1]
  ids, mask = ba._left_pad(np.array([], np.int32), 2, 9)
  assert ids.tolist() == [9, 9] and mask.tolist() == [0, 0]
  vals, mask = ba._right_pad([1.5, 2.5], 4, -1.0, np.float32)
  assert vals.tolist() == [1.5, 2.5, -1.0, -1.0] and mask.tolist() == [1, 1, 0, 0]
  vals, mask = ba._right_pad([1, 2, 3, 4, 5], 3, 0, np.int32)                    # the head survives
  assert vals.tolist() == [1, 2, 3] and mask.tolist() == [1, 1, 1]
  assert ba._right_pad([], 2, 7, np.int32)[0].tolist() == [7, 7]


def test_completion_aligned_values():
  assert ba._completion_aligned([1, 2], kept=2, length=4).tolist() == [1, 2, 0, 0]
  assert ba._completion_aligned(None, kept=2, length=3, fill_value=-1).tolist() == [-1, -1, -1]
  assert ba._completion_aligned(0.5, kept=3, length=4).tolist() == [0.5, 0.5, 0.5, 0]    # a scalar covers the kept tokens
  # values given over prompt + completion lose their prompt part
  assert ba._completion_aligned([9, 9, 1, 2, 3], kept=3, length=4, prompt_len=2).tolist() == [1, 2, 3, 0]
  # ... also when the completion itself was cut
  assert ba._completion_aligned([9, 1, 2, 3], kept=2, length=2, prompt_len=1, full_completion_len=3).tolist() == [1, 2]


def test_reference_logps_are_checked_before_they_are_attached():
  batch = ba.GRPOTrainExampleAssembler(batch_size=2, max_prompt_length=3, max_response_length=4, pad_id=0).pack(
      [grpo_item([1, 2], [3, 4, 5])])[0]
  ref = np.arange(8, dtype=np.float32).reshape(2, 4)
  assert ba.with_ref_per_token_logps(batch, ref).ref_per_token_logps.tolist() == ref.tolist()
  assert batch.ref_per_token_logps is None                                              # a new object, not a mutation
  answer = datatypes.LogprobsResponse(per_token_logps=ref)
  assert ba.with_ref_per_token_logps(batch, answer).ref_per_token_logps.dtype == np.float32
  failed = datatypes.LogprobsResponse(per_token_logps=ref, error=datatypes.ErrorInfo(error_type="X", message="scorer died"))
  with pytest.raises(RuntimeError, match="scorer died"):
    ba.with_ref_per_token_logps(batch, failed)
  with pytest.raises(ValueError, match=r"got \(2, 3\), expected \(2, 4\)"):
    ba.with_ref_per_token_logps(batch, ref[:, :3])
  with pytest.raises(TypeError, match="expects a padded TrainExample"):
    ba.with_ref_per_token_logps(payload([1, 2]), ref)


# ---- GRPO assembler -----------------------------------------------------------------------------------
def test_grpo_layout_truncation_and_filler_rows():
  asm = ba.GRPOTrainExampleAssembler(batch_size=3, max_prompt_length=3, max_response_length=3, pad_id=0)
  assert asm.pack([]) == []
  out = asm.pack([grpo_item([1, 2], [3, 4], adv=0.5), grpo_item([1, 2, 3, 4], [5, 6, 7, 8], adv=-2.0)])
  assert len(out) == 1 and isinstance(out[0], rl_common.TrainExample)
  ex = out[0]
  assert ex.prompt_ids.tolist() == [[0, 1, 2], [2, 3, 4], [0, 0, 0]]                    # left-padded, long prompts keep their tail
  assert ex.prompt_mask.tolist() == [[False, True, True], [True, True, True], [False] * 3]
  assert ex.completion_ids.tolist() == [[3, 4, 0], [5, 6, 7], [0, 0, 0]]                # right-padded, cut on the right
  assert ex.completion_mask.tolist() == [[True, True, False], [True, True, True], [False] * 3]
  assert ex.advantages.tolist() == [0.5, -2.0, 0.0]                                     # one per sequence; the filler row is inert
  assert ex.ref_per_token_logps is None and ex.old_per_token_logps is None
  with pytest.raises(ValueError, match="must be positive"):
    ba.GRPOTrainExampleAssembler(batch_size=0, max_prompt_length=1, max_response_length=1, pad_id=0)


def test_grpo_optional_fields_and_per_token_advantages():
  asm = ba.GRPOTrainExampleAssembler(batch_size=2, max_prompt_length=2, max_response_length=3, pad_id=0)
  a = grpo_item([1], [2, 3], adv=np.array([0.1, 0.2]), old_per_token_logps=np.array([-1.0, -2.0]),
                ref_per_token_logps=np.array([9.0, -3.0, -4.0]))                        # ref over prompt + completion
  b = grpo_item([1], [2, 3, 4], adv=np.array([0.3, 0.3, 0.3]))
  ex = asm.pack([a, b])[0]
  assert ex.old_per_token_logps.tolist() == [[-1.0, -2.0, 0.0], [0.0, 0.0, 0.0]]        # rows without the field: zeros
  assert ex.ref_per_token_logps.tolist() == [[-3.0, -4.0, 0.0], [0.0, 0.0, 0.0]]
  assert np.allclose(ex.advantages, [[0.1, 0.2, 0.0], [0.3, 0.3, 0.3]])                 # token-level values are kept as such
  masked = grpo_item([1], [2, 3, 4], completion_mask=np.array([1, 0, 1]))
  assert asm.pack([masked])[0].completion_mask.tolist()[0] == [True, False, True]


def test_grpo_chunks_into_micro_batches_of_equal_shape():
  asm = ba.GRPOTrainExampleAssembler(batch_size=2, max_prompt_length=2, max_response_length=2, pad_id=0)
  out = asm.pack([grpo_item([k], [k, k], adv=float(k)) for k in range(1, 6)])
  assert len(out) == 3 and all(ex.completion_ids.shape == (2, 2) for ex in out)
  assert [ex.advantages.tolist() for ex in out] == [[1.0, 2.0], [3.0, 4.0], [5.0, 0.0]]


# ---- token-stream assemblers --------------------------------------------------------------------------
def test_rectangular_batches_have_static_shape_and_masked_filler_rows():
  asm = ba.PaddedBatchAssembler(batch_size=2, max_seq_len=5, pad_id=9)
  assert asm.pack([]) == [] and asm.max_seq_len == asm.max_len == 5
  out = asm.pack([payload([1, 2, 3], loss=[0, 1, 1], adv=2.0), payload([4, 5, 6, 7, 8, 9, 10]), payload([11])])
  assert len(out) == 2 and all(p.token_ids.shape == (2, 5) for p in out)
  first, second = out
  assert first.token_ids.tolist() == [[1, 2, 3, 9, 9], [4, 5, 6, 7, 8]]                 # right-padded; cut on the right
  assert first.token_mask.tolist() == [[1, 1, 1, 0, 0], [1, 1, 1, 1, 1]]
  assert first.advantages.tolist() == [[0, 2, 2, 0, 0], [1, 1, 1, 1, 1]]                # a scalar spreads over loss tokens
  assert second.token_ids.tolist() == [[11, 9, 9, 9, 9], [9, 9, 9, 9, 9]]
  assert second.token_mask[1].sum() == 0 and second.loss_mask[1].sum() == 0             # the filler row trains nothing
  for bad in (dict(batch_size=0), dict(max_seq_len=0)):
    with pytest.raises(ValueError, match="must be positive"):
      ba.PaddedBatchAssembler(**bad)


def test_action_mask_optional_fields_and_missing_advantages_in_rectangular_batches():
  asm = ba.PaddedBatchAssembler(batch_size=2, max_seq_len=4)
  tool_turn = payload([1, 2, 3, 4], loss=[0, 1, 1, 1], action_mask=np.array([0, 1, 0, 1]),         # token 3: an observation
                      returns=np.array([0.1, 0.2, 0.3, 0.4]), old_per_token_logps=np.array([-1.0, -2.0]),
                      prompt_ids=np.array([77, 78]), completion_ids=np.array([79]))
  plain = payload([5, 6], adv=None)
  out = asm.pack([tool_turn, plain])[0]
  assert out.action_mask.tolist() == [[0, 1, 0, 1], [1, 1, 0, 0]]                       # falls back to the loss mask
  assert out.returns.tolist()[0] == pytest.approx([0.1, 0.2, 0.3, 0.4]) and out.returns.tolist()[1] == [0, 0, 0, 0]
  assert out.old_per_token_logps.tolist() == [[-1.0, -2.0, 0.0, 0.0], [0.0] * 4]        # short fields are zero-extended
  assert out.advantages.tolist()[1] == [0, 0, 0, 0]
  assert out.ref_per_token_logps is None and out.old_values is None and out.sampler_is_weights is None
  assert out.prompt_ids is None and out.completion_ids is None                          # stream assemblers ignore them
  everything = payload([1, 2], ref_per_token_logps=[1, 2], old_per_token_logps=[3, 4], returns=[5, 6],
                       old_values=[7, 8], sampler_is_weights=[9, 10])
  full = asm.pack([everything])[0]
  for name, want in (("ref_per_token_logps", [1, 2]), ("old_per_token_logps", [3, 4]), ("returns", [5, 6]),
                     ("old_values", [7, 8]), ("sampler_is_weights", [9, 10])):
    assert getattr(full, name)[0, :2].tolist() == want and getattr(full, name)[1].sum() == 0, name


def test_sequence_packing_places_whole_streams_with_segments_and_fields():
  asm = ba.SequencePackedBatchAssembler(max_packed_len=6, pad_id=0)
  assert asm.pack([]) == []
  items = [payload([1, 1, 1], adv=1.0, returns=[0.1, 0.2, 0.3]), payload([2, 2, 2, 2], loss=[0, 1, 1, 1], adv=2.0),
           payload([3, 3], adv=3.0), payload([4] * 8, adv=4.0)]
  rows = asm.pack(items)
  assert all(r.token_ids.shape == (1, 6) for r in rows)
  # first-fit decreasing: the 8-token stream (cut to 6) fills a row; 4 + 2 share one; 3 gets the last
  assert [r.token_ids[0].tolist() for r in rows] == [[4] * 6, [2, 2, 2, 2, 3, 3], [1, 1, 1, 0, 0, 0]]
  mixed = rows[1]
  assert mixed.segment_ids[0].tolist() == [1, 1, 1, 1, 2, 2] and mixed.segment_positions[0].tolist() == [0, 1, 2, 3, 0, 1]
  assert mixed.loss_mask[0].tolist() == [0, 1, 1, 1, 1, 1] and mixed.advantages[0].tolist() == [0, 2, 2, 2, 3, 3]
  assert mixed.returns is None and rows[2].returns[0, :3].tolist() == pytest.approx([0.1, 0.2, 0.3])
  assert rows[2].segment_ids[0].tolist() == [1, 1, 1, 0, 0, 0] and rows[2].token_mask[0].tolist() == [1, 1, 1, 0, 0, 0]
  with pytest.raises(ValueError, match="must be positive"):
    ba.SequencePackedBatchAssembler(max_packed_len=0)
