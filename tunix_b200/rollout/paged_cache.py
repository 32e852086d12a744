"""Paged KV cache: fixed-size pages handed out from a free list, with reference counts so that
sequences sampled from one prompt share the prompt's full pages.

Per layer the cache is two tensors [num_pages, page_size, Kh, H]. A sequence is a list of page
ids; token t lives in page `pages[t // page_size]`, row `t % page_size`.
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence

import torch


class OutOfPages(RuntimeError):
  pass


class PageAllocator:
  def __init__(self, num_pages: int):
    self.num_pages = num_pages
    self._free: List[int] = list(range(num_pages - 1, -1, -1))
    self._ref = [0] * num_pages

  @property
  def free_pages(self) -> int:
    return len(self._free)

  def alloc(self, n: int) -> List[int]:
    if n > len(self._free):
      raise OutOfPages(f"need {n} pages, {len(self._free)} free")
    out = [self._free.pop() for _ in range(n)]
    for p in out:
      self._ref[p] = 1
    return out

  def share(self, pages: Sequence[int]) -> List[int]:
    for p in pages:
      assert self._ref[p] > 0, f"page {p} is not allocated"
      self._ref[p] += 1
    return list(pages)

  def free(self, pages: Sequence[int]) -> None:
    for p in pages:
      assert self._ref[p] > 0, f"double free of page {p}"
      self._ref[p] -= 1
      if self._ref[p] == 0:
        self._free.append(p)

  def refcount(self, page: int) -> int:
    return self._ref[page]


@dataclasses.dataclass
class PagedLayerCache:
  """What one attention layer needs for one forward pass over a paged cache.

  mode "prefill": the T new tokens of each row attend causally among themselves (a prompt with
  no earlier context) and their K/V rows are written to `slots`.
  mode "decode": one new token per row; it is written to its slot and attends to the
  `seq_lens[b]` tokens (itself included) found through `block_tables[b]`.
  """
  k_pages: torch.Tensor
  v_pages: torch.Tensor
  slots: torch.Tensor            # int64 [B*T], -1 = do not store
  block_tables: torch.Tensor     # int32 [B, max_blocks]
  seq_lens: torch.Tensor         # int32 [B], lengths after this step's write
  mode: str = "decode"
  num_splits: Optional[int] = None
  max_len: Optional[int] = None


class PagedKVCache:
  def __init__(self, num_layers: int, num_pages: int, page_size: int, num_kv_heads: int, head_dim: int,
               dtype: torch.dtype, device):
    self.page_size, self.num_pages = page_size, num_pages
    shape = (num_pages, page_size, num_kv_heads, head_dim)
    self.k = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
    self.v = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(num_layers)]
    self.allocator = PageAllocator(num_pages)

  def pages_for(self, n_tokens: int) -> int:
    return (n_tokens + self.page_size - 1) // self.page_size

  def layer_caches(self, slots, block_tables, seq_lens, mode: str, num_splits=None, max_len=None
                   ) -> Dict[str, PagedLayerCache]:
    return {f"layer_{i}": PagedLayerCache(self.k[i], self.v[i], slots, block_tables, seq_lens, mode, num_splits,
                                          max_len) for i in range(len(self.k))}

  def copy_page(self, src: int, dst: int, rows: int) -> None:
    """Copies the first `rows` rows of page `src` to page `dst` in every layer (tail page of a
    shared prompt, which each sample must own because it appends to it)."""
    for k, v in zip(self.k, self.v):
      k[dst, :rows].copy_(k[src, :rows])
      v[dst, :rows].copy_(v[src, :rows])

  def bytes(self) -> int:
    return sum(t.numel() * t.element_size() for t in self.k) * 2
