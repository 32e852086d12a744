"""`generate/utils.py`: small helpers, decoding masks, output padding, parallelism sizes, and weight transfer through
a key mapping (wildcards, transposes, hooks, KV-head repetition, head-dim padding, dtype casts, tied heads) or by
structure (KV repetition inside stacked layers, casting, aliasing when buffers are dropped)."""
import numpy as np
import pytest
import torch

from tunix_b200.generate import utils as gu


def test_small_helpers():
  assert [gu.next_power_of_2(x) for x in (-3, 0, 1, 2, 3, 8, 9, 1000)] == [1, 1, 1, 2, 4, 8, 16, 1024]
  ids = np.array([0, 0, 5, 6, 0])
  assert gu.np_find_first_non_pad_idx(ids, 0) == 2 and gu.np_find_first_non_pad_idx(np.zeros(3, int), 0) == 0
  assert gu.np_find_first_eos_idx(np.array([4, 2, 9, 2]), [2]) == 1
  assert gu.np_find_first_eos_idx(np.array([4, 7]), [2, 9]) == 2                      # none: the whole row
  assert gu.find_first_eos_idx(torch.tensor([4, 9, 2]), [2, 9]) == 1
  assert gu.pad_to_length(np.array([1, 2]), 4, -1).tolist() == [1, 2, -1, -1]
  assert gu.pad_to_length(np.array([1, 2]), 4, -1, left=True).tolist() == [-1, -1, 1, 2]
  grid = np.arange(4).reshape(2, 2)
  assert gu.pad_to_length(grid, 3, 0, axis=1).tolist() == [[0, 1, 0], [2, 3, 0]] and gu.pad_to_length(grid, 1) is grid


def test_decoding_masks():
  valid = torch.tensor([[False, True, True], [True, True, True]])
  pre = gu.make_prefill_attention_mask(valid, cache_size=5)
  assert pre.shape == (2, 3, 5)
  assert pre[0].int().tolist() == [[0, 0, 0, 0, 0], [0, 1, 0, 0, 0], [0, 1, 1, 0, 0]]        # causal, blind to padding
  assert pre[1].int().tolist() == [[1, 0, 0, 0, 0], [1, 1, 0, 0, 0], [1, 1, 1, 0, 0]]
  buffer_valid = torch.tensor([[False, True, True, True, True], [True] * 5])
  dec = gu.make_decode_attention_mask(buffer_valid, step=3, cache_size=6)
  assert dec.shape == (2, 1, 6) and dec[0, 0].int().tolist() == [0, 1, 1, 1, 0, 0] and dec[1, 0].int().tolist() == [1, 1, 1, 1, 0, 0]


def test_padded_outputs_cut_at_eos_and_optionally_echo_the_prompt():
  P = 3
  buffers = np.array([[0, 5, 6, 7, 8, 2, 9], [4, 5, 6, 7, 8, 9, 9]])                     # pad 0, eos 2
  logits = np.arange(2 * 7 * 2, dtype=np.float32).reshape(2, 7, 2)
  lengths, toks, lg = gu.padded_fill_tokens_and_logits(buffers, logits, True, False, 0, [2], P, 4)
  assert lengths.tolist() == [2, 4] and toks.tolist() == [[7, 8, 0, 0], [7, 8, 9, 9]]
  assert lg.shape == (2, 4, 2) and lg[0, :2].tolist() == logits[0, 3:5].tolist() and not lg[0, 2:].any()
  lengths, toks, lg = gu.padded_fill_tokens_and_logits(buffers, None, False, True, 0, [2], P, 7)
  assert lengths.tolist() == [4, 7] and toks[0].tolist() == [5, 6, 7, 8, 0, 0, 0] and lg is None


@pytest.mark.parametrize("args, want", [((8,), (8, 1, 1)), ((8, 2), (2, 4, 1)), ((8, -1, 2), (4, 2, 1)),
                                        ((8, 4, 2, 4), (4, 2, 4))])
def test_parallelism_sizes_are_completed(args, want):
  assert gu.resolve_parallelism_sizes(*args) == want


def test_parallelism_sizes_that_do_not_fit_are_refused():
  for bad in ((8, 3), (8, -1, 3), (8, 2, 2)):
    with pytest.raises(ValueError):
      gu.resolve_parallelism_sizes(*bad)


# ---- transfer through a mapping ------------------------------------------------------------------------
def test_mapped_transfer_with_wildcards_transposes_hooks_and_casts():
  torch.manual_seed(0)
  src = {"tok.embed": torch.randn(10, 4), "blocks.0.attn.wq": torch.randn(4, 8), "blocks.1.attn.wq": torch.randn(4, 8),
         "blocks.0.norm": torch.randn(4), "blocks.1.norm": torch.randn(4), "unused.extra": torch.randn(2)}
  dst = {"embedder.w": torch.zeros(10, 4, dtype=torch.bfloat16), "layers.0.q.w": torch.zeros(8, 4),
         "layers.1.q.w": torch.zeros(8, 4), "layers.0.ln": torch.zeros(4), "layers.1.ln": torch.zeros(4)}
  mapping = {"tok.embed": ("embedder.w", None), "blocks.*.attn.wq": ("layers.*.q.w", "spec-q"),
             "blocks.*.norm": ("layers.*.ln", None)}
  seen_specs = []
  out = gu.transfer_state_with_mappings(src, dst, mapping, transpose_keys={"attn.wq": (1, 0)},
                                        key_mapping_hook_fns={r"\.norm$": lambda v: v + 1.0},
                                        reshard_fn=lambda v, spec: (seen_specs.append(spec), v)[1])
  assert out is dst
  assert torch.equal(dst["embedder.w"], src["tok.embed"].bfloat16())                         # cast to the destination's dtype
  for i in range(2):
    assert torch.equal(dst[f"layers.{i}.q.w"], src[f"blocks.{i}.attn.wq"].t())
    assert torch.equal(dst[f"layers.{i}.ln"], src[f"blocks.{i}.norm"] + 1.0)
  assert seen_specs.count("spec-q") == 2 and len(seen_specs) == 5
  with pytest.raises(KeyError, match="no mapping produces destination keys"):
    gu.transfer_state_with_mappings(src, {**dst, "orphan": torch.zeros(1)}, mapping)
  with pytest.raises(KeyError, match="source state has no key"):
    gu.transfer_state_with_mappings({k: v for k, v in src.items() if k != "blocks.1.norm"}, dst, mapping,
                                    transpose_keys={"attn.wq": (1, 0)})


def test_kv_heads_are_repeated_and_head_dims_zero_padded_but_other_weights_are_not_stretched():
  k = torch.arange(2 * 3 * 4, dtype=torch.float32).view(2, 3, 4)                  # [kv heads, model dim, head dim]
  rep = gu._align_shape(k, (4, 3, 4), "layers.0.attn.k_proj.w")
  assert rep.shape == (4, 3, 4) and torch.equal(rep[0], rep[1]) and torch.equal(rep[2], rep[3]) and torch.equal(rep[2], k[1])
  padded = gu._align_shape(k, (2, 3, 6), "layers.0.attn.k_proj.w")                # last axis: head-dim padding with zeros
  assert torch.equal(padded[..., :4], k) and not padded[..., 4:].any()
  both = gu._align_shape(k, (4, 3, 6), "layers.0.attn.v_proj.w")
  assert both.shape == (4, 3, 6) and torch.equal(both[1, :, :4], k[0])
  plain = gu._align_shape(torch.ones(2, 3), (4, 3), "layers.0.mlp.up.w")         # not attention: padded, never repeated
  assert plain[:2].eq(1).all() and not plain[2:].any()
  assert gu._align_shape(k, (2, 3, 4), "anything") is k
  with pytest.raises(ValueError, match="rank mismatch"):
    gu._align_shape(k, (2, 12), "layers.0.attn.k_proj.w")
  with pytest.raises(ValueError, match="cannot align"):
    gu._align_shape(k, (1, 3, 4), "layers.0.attn.k_proj.w")                        # shrinking loses weights


def test_a_tied_head_follows_the_embedding():
  """The head is mapped like any key, and then overwritten from the embedding it is declared tied to (transposed
  when the head is stored the other way round)."""
  src = {"emb": torch.randn(6, 3)}
  for head_shape, expect in (((6, 3), lambda e: e), ((3, 6), lambda e: e.t())):
    dst = {"embedder.w": torch.zeros(6, 3), "lm_head.w": torch.zeros(head_shape)}
    with pytest.raises(KeyError):
      gu.transfer_state_with_mappings(src, dst, {"emb": ("embedder.w", None)})     # an unmapped key is still an error
    mapping = {"emb": ("embedder.w", None), "head": ("lm_head.w", None)}
    gu.transfer_state_with_mappings({**src, "head": torch.zeros(head_shape)}, dst, mapping,
                                    tie_lm_head=("embedder.w", "lm_head.w"))
    assert torch.equal(dst["lm_head.w"], expect(src["emb"]))


# ---- transfer by structure --------------------------------------------------------------------------
def test_direct_transfer_repeats_kv_heads_inside_stacked_layers_and_casts():
  torch.manual_seed(1)
  L = 2
  src = {"layers": {"attn": {"k_proj": {"w": torch.randn(L, 2, 3, 4)}}, "norm": {"w": torch.randn(L, 3)}}}
  dst = {f"layers.{i}.attn.k_proj.w": torch.zeros(4, 3, 4, dtype=torch.bfloat16) for i in range(L)}
  dst.update({f"layers.{i}.norm.w": torch.zeros(3, dtype=torch.float64) for i in range(L)})
  gu.transfer_state_directly(src, dst)
  for i in range(L):
    k = src["layers"]["attn"]["k_proj"]["w"][i]
    assert torch.equal(dst[f"layers.{i}.attn.k_proj.w"], k.repeat_interleave(2, 0).bfloat16())
    assert torch.equal(dst[f"layers.{i}.norm.w"], src["layers"]["norm"]["w"][i].double())


def test_direct_transfer_intersects_keys_and_leaves_aliased_buffers_alone():
  shared = torch.randn(3)
  src = {"a": shared, "b": torch.ones(2), "only_src": torch.ones(1)}
  dst = {"a": shared, "b": torch.zeros(2), "only_dst": torch.full((1,), 7.0)}
  before = dst["b"]
  gu.transfer_state_directly(src, dst, delete_dst_buffers=True)
  assert dst["a"] is shared and torch.equal(dst["a"], shared)                     # source and destination are one buffer
  assert before.eq(1).all() and dst["only_dst"].item() == 7.0
  assert gu.verify_state_closeness({"x": torch.ones(2)}, {"x": torch.ones(2) + 1e-3})
  assert not gu.verify_state_closeness({"x": torch.ones(2)}, {"x": torch.ones(2) + 0.1})
  assert not gu.verify_state_closeness({"x": torch.ones(2)}, {"y": torch.ones(2)})
