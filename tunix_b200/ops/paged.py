"""Paged KV cache operations and token sampling for the rollout engine.

CUDA bf16 tensors go to the kernels of `csrc/decode.cu`; anything else (CPU tests, fp32) runs
the plain PyTorch statement of the same operation below, which is also the test oracle.

Cache layout: `k_pages`, `v_pages` [num_pages, page_size, Kh, H]; `block_tables` [B, max_blocks]
int32 page ids per sequence; `seq_lens` [B] int32; `slots` [T] int64 = page * page_size + row.
"""
from __future__ import annotations

import math
import os
from typing import Optional, Sequence, Tuple

import torch

from . import _lib


def _use_kernels(*ts: torch.Tensor) -> bool:
  return all(t.is_cuda for t in ts) and ts[0].dtype == torch.bfloat16 and _lib.available()


# ---- KV write --------------------------------------------------------------------------------
def kv_page_write_ref(k_new, v_new, slots, k_pages, v_pages) -> None:
  P, page, Kh, H = k_pages.shape
  keep = slots >= 0
  idx = slots[keep]
  k_pages.view(P * page, Kh, H)[idx] = k_new[keep].to(k_pages.dtype)
  v_pages.view(P * page, Kh, H)[idx] = v_new[keep].to(v_pages.dtype)


def kv_page_write(k_new: torch.Tensor, v_new: torch.Tensor, slots: torch.Tensor, k_pages: torch.Tensor,
                  v_pages: torch.Tensor) -> None:
  """k_new / v_new [T, Kh, H] (may be strided views with contiguous heads) -> pages, in place."""
  T, Kh, H = k_new.shape
  if not _use_kernels(k_new, k_pages) or k_new.stride(2) != 1 or k_new.stride(1) != H or v_new.stride(1) != H:
    kv_page_write_ref(k_new, v_new, slots, k_pages, v_pages)
    return
  rc = _lib.require().tx_kv_page_write(k_new.data_ptr(), v_new.data_ptr(), k_new.stride(0), v_new.stride(0),
                                       slots.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), T, Kh, H,
                                       _lib.stream_ptr())
  _lib.check_rc(rc, "tx_kv_page_write")


# ---- decode attention ------------------------------------------------------------------------
def paged_decode_attention_ref(q, k_pages, v_pages, block_tables, seq_lens, scale: float) -> torch.Tensor:
  B, N, H = q.shape
  P, page, Kh, _ = k_pages.shape
  G = N // Kh
  out = torch.zeros(B, N, H, dtype=torch.float32, device=q.device)
  for b in range(B):
    n = int(seq_lens[b])
    if n == 0:
      continue
    pages = block_tables[b, :(n + page - 1) // page].long()
    k = k_pages[pages].reshape(-1, Kh, H)[:n].float()
    v = v_pages[pages].reshape(-1, Kh, H)[:n].float()
    qb = q[b].float().view(Kh, G, H)
    s = torch.einsum("kgh,tkh->kgt", qb, k) * scale
    out[b] = torch.einsum("kgt,tkh->kgh", torch.softmax(s, -1), v).reshape(N, H)
  return out.to(q.dtype)


_ws = {}


def _workspace(device, n_o: int, n_ml: int) -> Tuple[torch.Tensor, torch.Tensor]:
  key = (device.index, torch.cuda.is_current_stream_capturing())
  cur = _ws.get(key)
  if cur is None or cur[0].numel() < n_o or cur[1].numel() < n_ml:
    cur = (torch.empty(n_o, dtype=torch.float32, device=device), torch.empty(n_ml, dtype=torch.float32, device=device))
    _ws[key] = cur
  return cur


def choose_splits(batch: int, kv_heads: int, max_len: int, sm_count: int = 148) -> int:
  """Enough CTAs to fill the GPU twice over, but at least 256 keys per split."""
  want = max(1, (2 * sm_count + batch * kv_heads - 1) // (batch * kv_heads))
  return int(max(1, min(want, max_len // 256, 32)))


def tc_supported(head_dim: int, page_size: int, group: int) -> bool:
  """Shapes the tensor-core decode kernel covers; TUNIX_B200_DECODE_TC=0 forces the SIMT kernel."""
  return (head_dim == 128 and page_size in (8, 16, 32, 64) and 1 <= group <= 32
          and os.environ.get("TUNIX_B200_DECODE_TC", "1") != "0")


def paged_decode_attention(q: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor, block_tables: torch.Tensor,
                           seq_lens: torch.Tensor, scale: float, num_splits: Optional[int] = None,
                           max_len: Optional[int] = None) -> torch.Tensor:
  """q [B, N, H] -> [B, N, H]: each row attends to the `seq_lens[b]` cached tokens of its pages."""
  B, N, H = q.shape
  P, page, Kh, _ = k_pages.shape
  tc = tc_supported(H, page, N // Kh)
  if (not _use_kernels(q, k_pages) or H not in (64, 128, 256) or (N // Kh > 8 and not tc) or q.stride(2) != 1
      or q.stride(1) != H):
    return paged_decode_attention_ref(q, k_pages, v_pages, block_tables, seq_lens, scale)
  if num_splits is None:
    num_splits = choose_splits(B, Kh, max_len if max_len is not None else block_tables.shape[1] * page)
  out = torch.empty((B, N, H), dtype=q.dtype, device=q.device)
  ws_o = ws_ml = None
  if num_splits > 1:
    ws_o, ws_ml = _workspace(q.device, B * N * num_splits * H, B * N * num_splits * 2)
  lib = _lib.require()
  if tc and k_pages.is_contiguous() and v_pages.is_contiguous():
    rc = lib.tx_paged_decode_attn_tc(
        q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), block_tables.data_ptr(),
        block_tables.stride(0), seq_lens.data_ptr(), B, N, Kh, H, page, P, float(scale), int(num_splits),
        ws_o.data_ptr() if ws_o is not None else None, ws_ml.data_ptr() if ws_ml is not None else None,
        out.data_ptr(), out.stride(0), _lib.status_word(q.device).data_ptr(), _lib.stream_ptr())
    _lib.check_rc(rc, "tx_paged_decode_attn_tc")
    if num_splits > 1:
      _lib.check_rc(lib.tx_paged_decode_combine(ws_o.data_ptr(), ws_ml.data_ptr(), int(num_splits), out.data_ptr(),
                                                out.stride(0), B, N, H, _lib.stream_ptr()),
                    "tx_paged_decode_combine")
    return out
  rc = lib.tx_paged_decode_attn(
      q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(), block_tables.data_ptr(),
      block_tables.stride(0), seq_lens.data_ptr(), B, N, Kh, H, page, float(scale), int(num_splits),
      ws_o.data_ptr() if ws_o is not None else None, ws_ml.data_ptr() if ws_ml is not None else None, out.data_ptr(),
      out.stride(0), _lib.stream_ptr())
  _lib.check_rc(rc, "tx_paged_decode_attn")
  return out


# ---- sampling --------------------------------------------------------------------------------
def sample_ref(logits: torch.Tensor, temperature: float, greedy: bool, generator: Optional[torch.Generator] = None,
               forbidden: Optional[Sequence[int]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
  z = logits.float() * (1.0 if greedy else 1.0 / temperature)
  if forbidden:
    z = z.clone()
    z[:, list(forbidden)] = float("-inf")
  lp = torch.log_softmax(z, -1)
  if greedy:
    tok = torch.argmax(z, -1)
  else:
    tok = torch.multinomial(lp.exp(), 1, generator=generator).squeeze(-1)
  return tok, lp.gather(-1, tok[:, None]).squeeze(-1)


def sample_filtered_ref(logits: torch.Tensor, temperature: float, top_k: Optional[int], top_p: Optional[float],
                        generator: Optional[torch.Generator] = None,
                        forbidden: Optional[Sequence[int]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
  """Top-k then top-p over the sorted candidates, categorical draw among the survivors; the log-prob is
  that of the drawn token under the full tempered softmax (tunix/generate/sampler.py:105-161)."""
  z = logits.float() / temperature
  if forbidden:
    z = z.clone()
    z[:, list(forbidden)] = float("-inf")
  k = z.shape[-1] if not top_k or top_k <= 0 else min(int(top_k), z.shape[-1])
  zs, idx = torch.topk(z, k, dim=-1)
  if top_p is not None and top_p < 1.0:
    ps = torch.softmax(zs, dim=-1)
    zs = torch.where(torch.cumsum(ps, dim=-1) - ps > top_p, torch.full_like(zs, float("-inf")), zs)
  pick = torch.multinomial(torch.softmax(zs, -1), 1, generator=generator)
  tok = idx.gather(-1, pick).squeeze(-1)
  lp = torch.log_softmax(z, -1).gather(-1, tok[:, None]).squeeze(-1)
  return tok, lp


def sample(logits: torch.Tensor, temperature: float = 1.0, greedy: bool = False, seed: int = 0,
           step: int = 0, step_tensor: Optional[torch.Tensor] = None, forbidden: Optional[torch.Tensor] = None,
           want_logprobs: bool = True, top_k: Optional[int] = None, top_p: Optional[float] = None,
           n_forbidden: Optional[int] = None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
  """logits [B, V] (fp32 or bf16, contiguous rows) -> (tokens int64 [B], logprobs fp32 [B]).

  Greedy, or an exact categorical draw from softmax(logits / temperature) (Gumbel-max with a
  counter-based generator keyed by seed and step), optionally restricted to the top-k / top-p
  candidates first - all inside one kernel launch. `step_tensor` (int64 scalar on the device)
  is added to `step`, so a captured CUDA graph can advance the stream of draws by bumping it.
  `forbidden` is an int32 tensor of token ids that are never chosen (`n_forbidden` of them when the
  tensor is a larger static buffer). The returned log-prob is that of the chosen token under the
  full (forbidden-masked) distribution at that temperature."""
  B, V = logits.shape
  filtered = not greedy and ((top_k is not None and 0 < top_k < V) or (top_p is not None and top_p < 1.0))
  nf = 0 if forbidden is None else (forbidden.numel() if n_forbidden is None else int(n_forbidden))
  if not (logits.is_cuda and _lib.available() and logits.dtype in (torch.float32, torch.bfloat16)
          and logits.stride(1) == 1):
    g = torch.Generator(device=logits.device)
    extra = int(step_tensor.item()) if step_tensor is not None else 0
    g.manual_seed((seed * 1_000_003 + (step + extra) * 7919 + 12345) % (2 ** 63 - 1))
    fl = forbidden[:nf].tolist() if nf else None
    if filtered:
      return sample_filtered_ref(logits, temperature, top_k, top_p, g, fl)
    return sample_ref(logits, temperature, greedy, g, fl)
  tokens = torch.empty(B, dtype=torch.int64, device=logits.device)
  lps = torch.empty(B, dtype=torch.float32, device=logits.device) if want_logprobs else None
  fptr = forbidden.data_ptr() if nf else None
  sptr = step_tensor.data_ptr() if step_tensor is not None else None
  if filtered:
    rc = _lib.require().tx_sample_filtered(
        logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0), B, V, float(temperature),
        int(top_k or 0), float(top_p if top_p is not None else 1.0), int(seed) & (2 ** 64 - 1), sptr, int(step), fptr,
        nf, tokens.data_ptr(), lps.data_ptr() if lps is not None else None, _lib.stream_ptr())
    _lib.check_rc(rc, "tx_sample_filtered")
    return tokens, lps
  rc = _lib.require().tx_sample(
      logits.data_ptr(), int(logits.dtype == torch.bfloat16), logits.stride(0), B, V, float(temperature), int(greedy),
      int(seed) & (2 ** 64 - 1), sptr, int(step), fptr, nf, tokens.data_ptr(),
      lps.data_ptr() if lps is not None else None, _lib.stream_ptr())
  _lib.check_rc(rc, "tx_sample")
  return tokens, lps
