"""`rl/common.py` against hand-written oracles: KL estimators and clamping, log-prob selection, id processing,
per-token log-probs (padding, temperature, entropy, packed rows), completion masks, padding, and every loss
aggregation mode - plain, packed, in bf16, and through the reducers."""
import math

import numpy as np
import pytest
import torch

from tunix_b200.rl import common
from tests.test_rl_grpo import toy_model

MODES = ["token-mean", "sequence-mean-token-mean", "sequence-mean-token-scale", "seq-mean-token-sum",
         "sequence-mean-token-sum-norm"]


# ---- KL ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("method", ["kl", "mse_kl", "low_var_kl"])
def test_kl_estimators_match_their_formulas_and_vanish_at_equality(method):
  g = torch.Generator().manual_seed(0)
  lp, ref = -torch.rand(3, 5, generator=g) * 4, -torch.rand(3, 5, generator=g) * 4
  got = common.compute_kl_divergence(lp, ref, method)
  for b in range(3):
    for t in range(5):
      a, r = float(lp[b, t]), float(ref[b, t])
      want = {"kl": a - r, "mse_kl": 0.5 * (a - r) ** 2, "low_var_kl": math.exp(r - a) - (r - a) - 1}[method]
      assert float(got[b, t]) == pytest.approx(want, rel=1e-5, abs=1e-6)
  assert common.compute_kl_divergence(lp, lp, method).abs().max() == 0
  if method != "kl":
    assert (got >= 0).all()                       # both are non-negative estimators


def test_kl_clamp_is_symmetric_and_a_no_op_by_default_and_in_range():
  lp = torch.tensor([[0.0, -10.0, -0.1]])
  ref = torch.tensor([[-10.0, 0.0, -0.2]])
  raw = common.compute_kl_divergence(lp, ref, "kl")
  assert raw.tolist() == [[10.0, -10.0, pytest.approx(0.1)]]
  clamped = common.compute_kl_divergence(lp, ref, "kl", clamp_value=2.0)
  assert clamped.tolist() == [[2.0, -2.0, pytest.approx(0.1)]]
  big = common.compute_kl_divergence(lp, ref, "low_var_kl", clamp_value=5.0)
  assert float(big.max()) == 5.0 and float(big[0, 2]) == pytest.approx(math.exp(-0.1) + 0.1 - 1, abs=1e-6)


def test_kl_in_bf16_is_computed_in_fp32():
  lp = torch.tensor([[-1.0, -2.5]], dtype=torch.bfloat16)
  ref = torch.tensor([[-1.5, -2.0]], dtype=torch.bfloat16)
  out = common.compute_kl_divergence(lp, ref, "low_var_kl")
  assert out.dtype == torch.float32
  torch.testing.assert_close(out, common.compute_kl_divergence(lp.float(), ref.float(), "low_var_kl"))


# ---- log-prob selection ----------------------------------------------------------------------------
def test_selective_log_softmax_and_entropy():
  logits = torch.tensor([[[1.0, 2.0, 3.0], [0.0, 0.0, 0.0]]])
  ids = torch.tensor([[2, 1]])
  got = common.selective_log_softmax(logits, ids)
  z = math.log(math.e + math.e ** 2 + math.e ** 3)
  assert got.tolist() == [[pytest.approx(3.0 - z, abs=1e-6), pytest.approx(-math.log(3.0), abs=1e-6)]]
  ent = common.compute_entropy_from_logits(logits)
  assert float(ent[0, 1]) == pytest.approx(math.log(3.0), abs=1e-6) and float(ent[0, 0]) < math.log(3.0)


def test_process_ids_positions_masks_and_the_packed_contract():
  prompt = torch.tensor([[0, 0, 5, 6], [0, 7, 8, 9]])
  completion = torch.tensor([[3, 2, 0], [4, 4, 2]])
  ids, pos, attn, seg = common.process_ids(prompt, completion, pad_id=0, eos_id=2)
  assert ids.tolist() == [[0, 0, 5, 6, 3, 2, 0], [0, 7, 8, 9, 4, 4, 2]]
  assert pos[0, 2:6].tolist() == [0, 1, 2, 3] and pos[1, 1:].tolist() == [0, 1, 2, 3, 4, 5]
  assert seg.tolist() == [[0, 0, 1, 1, 1, 1, 0], [0, 1, 1, 1, 1, 1, 1]]
  # causal and blind to padding: token 4 of row 0 sees columns 2..4 only
  row = attn[0, 4] if attn.dim() == 3 else attn[0, 0, 4]
  assert row.tolist() == [False, False, True, True, True, False, False]
  with pytest.raises(ValueError, match="segment_positions"):
    common.process_ids(prompt, completion, 0, 2, segment_ids=torch.ones(2, 7, dtype=torch.int32))
  packed = common.process_ids(prompt, completion, 0, 2, segment_ids=torch.ones(2, 7, dtype=torch.int32),
                              segment_positions=torch.arange(7).expand(2, 7))
  assert packed[2] is None and packed[3] is None and packed[1].shape == (2, 7)


def test_per_token_logps_against_a_direct_forward_pass():
  model = toy_model()
  g = torch.Generator().manual_seed(1)
  prompt = torch.randint(3, 64, (2, 5), generator=g)
  prompt[0, :2] = 0                                    # left padding
  completion = torch.randint(3, 64, (2, 4), generator=g)
  completion[1, 3] = 0                                 # right padding
  lp, ent = common.compute_per_token_logps(model, prompt, completion, pad_id=0, eos_id=2, return_entropy=True)
  assert lp.shape == (2, 4) and ent.shape == (2, 4) and not lp.requires_grad
  ids, pos, attn, _ = common.process_ids(prompt, completion, 0, 2)
  logits = model(ids, pos, None, attn)[0].float()
  want = torch.log_softmax(logits[:, 4:8], -1).gather(-1, completion[..., None])[..., 0]
  torch.testing.assert_close(lp, want, rtol=1e-4, atol=1e-5)
  torch.testing.assert_close(ent, common.compute_entropy_from_logits(logits[:, 4:8]), rtol=1e-4, atol=1e-5)
  # padding in the prompt does not leak: the same row without its padding gives the same numbers
  alone = common.compute_per_token_logps(model, prompt[:1, 2:], completion[:1], 0, 2)
  torch.testing.assert_close(alone, lp[:1], rtol=1e-4, atol=1e-5)
  # temperature divides the logits; gradients flow only when asked
  hot = common.compute_per_token_logps(model, prompt, completion, 0, 2, temperature=2.0)
  want_hot = torch.log_softmax(logits[:, 4:8] / 2.0, -1).gather(-1, completion[..., None])[..., 0]
  torch.testing.assert_close(hot, want_hot, rtol=1e-4, atol=1e-5)
  live = common.compute_per_token_logps(model, prompt, completion, 0, 2, stop_gradient=False)
  assert live.requires_grad
  old_api = common.get_per_token_logps(model, ids, pos, attn, logits_to_keep=4)
  torch.testing.assert_close(old_api, want, rtol=1e-4, atol=1e-5)


def test_packed_rows_give_each_segment_its_unpacked_logps():
  """Two sequences in one row (segment ids 1 and 2, positions restarting) score like the two rows alone."""
  model = toy_model()
  g = torch.Generator().manual_seed(2)
  a, b = torch.randint(3, 64, (1, 6), generator=g), torch.randint(3, 64, (1, 5), generator=g)
  row = torch.cat([a, b, torch.zeros(1, 2, dtype=torch.long)], dim=1)
  seg = torch.tensor([[1] * 6 + [2] * 5 + [0] * 2])
  pos = torch.tensor([list(range(6)) + list(range(5)) + [0, 0]])
  packed = common.compute_per_token_logps(model, row[:, :0], row, pad_id=0, eos_id=2, segment_ids=seg,
                                          segment_positions=pos)
  assert packed.shape == (1, 13) and float(packed[0, 0]) == 0.0          # left-padded: position t scores token t
  for seq, lo in ((a, 0), (b, 6)):
    alone = common.compute_per_token_logps(model, seq[:, :1], seq[:, 1:], pad_id=0, eos_id=2)
    torch.testing.assert_close(packed[:, lo + 1: lo + seq.shape[1]], alone, rtol=1e-4, atol=1e-5)


def test_model_call_contains_sees_names_kwargs_and_wrapped_models():
  class Plain(torch.nn.Module):
    def forward(self, tokens, positions): return tokens
  class Open(torch.nn.Module):
    def forward(self, tokens, **kw): return tokens
  class Wrapper:
    def __init__(self): self.transformer = Plain()
  assert common.model_call_contains(Plain(), "positions") and not common.model_call_contains(Plain(), "segment_ids")
  assert common.model_call_contains(Open(), "segment_ids") and common.model_call_contains(Wrapper(), "positions")
  assert common.model_call_contains(toy_model(), "segment_ids")


def test_compute_score_squeezes_and_ignores_segments_the_model_cannot_take():
  class Scorer(torch.nn.Module):
    def forward(self, tokens, positions, cache, attention_mask):
      return tokens.float()[..., None] * 0.5, None
  prompt, completion = torch.tensor([[0, 3, 4]]), torch.tensor([[5, 6]])
  out = common.compute_score(Scorer(), prompt, completion, pad_id=0, eos_id=2)
  assert out.tolist() == [[0.0, 1.5, 2.0, 2.5, 3.0]] and not out.requires_grad


# ---- masks and padding -------------------------------------------------------------------------------
def test_completion_masks_numpy_and_torch_agree():
  ids = np.array([[5, 2, 7, 2], [5, 6, 7, 8], [2, 2, 2, 2]])
  want = [[1, 1, 0, 0], [1, 1, 1, 1], [1, 0, 0, 0]]
  assert common.np_make_completion_mask(ids, eos_tok=2).tolist() == want
  assert common.make_completion_mask(torch.as_tensor(ids), eos_tok=2).tolist() == want


@pytest.mark.parametrize("kind", ["numpy", "torch"])
def test_pad_to_length_sides_axes_and_no_op(kind):
  x = np.arange(6).reshape(2, 3)
  x = x if kind == "numpy" else torch.as_tensor(x)
  assert common.pad_to_length(x, 4, -1, axis=0).tolist() == [[0, 1, 2], [3, 4, 5], [-1, -1, -1], [-1, -1, -1]]
  assert common.pad_to_length(x, 5, 9, left=True, axis=1).tolist() == [[9, 9, 0, 1, 2], [9, 9, 3, 4, 5]]
  assert common.pad_to_length(x, 2, 0, axis=1) is x


# ---- loss aggregation -----------------------------------------------------------------------------
LOSS = torch.tensor([[1.0, 2.0, 3.0, 4.0], [5.0, 6.0, 7.0, 8.0], [9.0, 9.0, 9.0, 9.0]])
MASK = torch.tensor([[1, 1, 0, 0], [1, 1, 1, 1], [0, 0, 0, 0]])


@pytest.mark.parametrize("mode, kwargs, want", [
    ("token-mean", {}, (1 + 2 + 5 + 6 + 7 + 8) / 6),
    ("sequence-mean-token-mean", {}, (1.5 + 6.5) / 2),                   # the empty row does not count
    ("sequence-mean-token-scale", {}, (3 / 4 + 26 / 4) / 2),             # norm defaults to the row width
    ("sequence-mean-token-scale", {"norm": 2.0}, (3 / 2 + 26 / 2) / 2),
    ("seq-mean-token-sum", {}, (3 + 26) / 2),
    ("sequence-mean-token-sum-norm", {}, 29 / 3),                        # norm defaults to the batch size
    ("sequence-mean-token-sum-norm", {"norm": 10}, 2.9),
])
def test_aggregation_modes_by_hand(mode, kwargs, want):
  metric = common.aggregate_loss(LOSS, MASK, mode, **kwargs)
  assert float(metric.compute()) == pytest.approx(want, rel=1e-6)
  assert float(common.reduced_loss_agg(LOSS, MASK, mode, **kwargs)) == pytest.approx(want, rel=1e-6)


@pytest.mark.parametrize("mode", MODES)
def test_aggregation_all_masked_is_zero_not_nan(mode):
  metric = common.aggregate_loss(LOSS, torch.zeros_like(MASK), mode)
  assert float(metric.compute()) == 0.0


@pytest.mark.parametrize("mode", MODES)
def test_packed_aggregation_equals_the_unpacked_batch(mode):
  """Rows 0 and 1 of the batch above packed into one row (segments 1 and 2, padding segment 0)."""
  packed = torch.tensor([[1.0, 2.0, 5.0, 6.0, 7.0, 8.0, 100.0, 100.0]])
  pmask = torch.tensor([[1, 1, 1, 1, 1, 1, 0, 0]])
  seg = torch.tensor([[1, 1, 2, 2, 2, 2, 0, 0]])
  kw = {"norm": 4.0} if mode == "sequence-mean-token-scale" else ({"norm": 3} if mode.endswith("sum-norm") else {})
  a = common.aggregate_loss(packed, pmask, mode, segment_ids=seg, num_segments=3, **kw)
  b = common.aggregate_loss(LOSS, MASK, mode, **kw)
  assert float(a.compute()) == pytest.approx(float(b.compute()), rel=1e-6)
  assert float(common.reduced_loss_agg(packed, pmask, mode, segment_ids=seg, num_segments=3, **kw)) == \
      pytest.approx(float(b.compute()), rel=1e-6)


def test_packed_aggregation_demands_what_it_cannot_guess():
  seg = torch.tensor([[1, 1, 0, 0]])
  with pytest.raises(ValueError, match="num_segments"):
    common.aggregate_loss(LOSS[:1], MASK[:1], "token-mean", segment_ids=seg)
  with pytest.raises(ValueError, match="explicit 'norm'"):
    common.aggregate_loss(LOSS[:1], MASK[:1], "sequence-mean-token-scale", segment_ids=seg, num_segments=2)


@pytest.mark.parametrize("norm", [0, -1, "x", None])
def test_invalid_norms_and_modes_are_rejected(norm):
  with pytest.raises(ValueError, match="norm"):
    common.aggregate_loss(LOSS, MASK, "sequence-mean-token-sum-norm", norm=norm)
  with pytest.raises(ValueError, match="Unsupported loss aggregation mode"):
    common.aggregate_loss(LOSS, MASK, "mean-of-everything")


def test_aggregation_in_bf16_accumulates_in_fp32():
  g = torch.Generator().manual_seed(0)
  loss = torch.rand(4, 512, generator=g)
  mask = torch.ones(4, 512)
  want = float(common.aggregate_loss(loss, mask, "token-mean").compute())
  got = common.aggregate_loss(loss.bfloat16(), mask.bfloat16(), "token-mean")
  assert got.unreduced_sum.dtype == torch.float32
  assert float(got.compute()) == pytest.approx(want, rel=4e-3)        # bf16 inputs, fp32 sum: no 2048-term drift


def test_micro_batch_reducers():
  """Summing numerators and denominators over micro-batches equals aggregating the whole batch at once; the mean of
  per-micro-batch means does not when the micro-batches hold different token counts."""
  parts = [common.aggregate_loss(LOSS[:1], MASK[:1], "token-mean"), common.aggregate_loss(LOSS[1:], MASK[1:], "token-mean")]
  whole = float(common.aggregate_loss(LOSS, MASK, "token-mean").compute())
  assert common.global_weighted_mean(parts) == pytest.approx(whole, rel=1e-6)
  assert float(common.mean_of_means(parts)) == pytest.approx((1.5 + 6.5) / 2, rel=1e-6) != pytest.approx(whole)
  assert float(common.mean_of_means([1.0, 2.0, 6.0])) == 3.0
  zero = [common.aggregate_loss(LOSS, torch.zeros_like(MASK), "seq-mean-token-sum")]
  assert common.global_weighted_mean(zero) == 0.0


def test_segment_helpers_drop_out_of_range_ids():
  values = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
  ids = torch.tensor([[0, 1, 1, 5]])
  assert common.segmented_sum(values, ids, 3).tolist() == [[1.0, 5.0, 0.0]]
  assert common.segmented_count(ids, 3).tolist() == [[1.0, 2.0, 0.0]]
  assert common.segmented_count(ids, 3, mask=torch.tensor([[1, 0, 1, 1]])).tolist() == [[1.0, 1.0, 0.0]]
