"""Checkpoint key translation by regular expressions (tunix/utils/torch_utils.py:5-18).

A mapping is {pattern: (replacement, layout hint)}: the key of a tensor in a foreign checkpoint must match exactly
one pattern (`re.match`, anchored at the start), and becomes `re.sub(pattern, replacement, key)` together with that
pattern's hint (a transpose permutation, a reshape, or None; what it means is up to the loader that owns the mapping).
Zero or several matches are both errors: a silent first-match rule would let an overly broad pattern load a tensor
into the wrong parameter.
"""
from __future__ import annotations

import re
from typing import Any, Mapping, Tuple


def map_checkpoint_key(mapping: Mapping[str, Tuple[str, Any]], source_key: str) -> Tuple[str, Any]:
  hits = [(re.sub(pattern, replacement, source_key), hint) for pattern, (replacement, hint) in mapping.items()
          if re.match(pattern, source_key)]
  if not hits:
    raise ValueError(f"no pattern of the mapping matches checkpoint key {source_key!r}")
  if len(hits) > 1:
    raise ValueError(f"{len(hits)} patterns match checkpoint key {source_key!r}: {[h[0] for h in hits]}")
  return hits[0]


torch_key_to_jax_key = map_checkpoint_key       # the reference's name for the same function
