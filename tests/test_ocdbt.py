"""OCDBT reader: a checkpoint written by Orbax (bytes embedded below) and round trips of the writer."""
import base64
import os

import numpy as np
import pytest
import torch

from tunix_b200.ckpt import ocdbt, orbax_layout

# A 2-layer toy model saved by Orbax with its default OCDBT + zarr(zstd) settings: w1/{bias [4], kernel [2,4]},
# w2/{bias [2], kernel [4,2]}, float32. Three files of the `model_params` item directory.
GOLDEN = {
    "manifest.ocdbt": (
        "DNs6KnEAAAAAAAAAAAEotS/9IFaxAgDQavJMoItfoUoRw7eDOCRgAIAIgMLXLwQBAAAAAAEiAGQvOGYyZWQ5ZDQ1ZWM4MWViYTlj"
        "NTYxMjA2NWVlNjY5NTgBAQAAAJYDEZYDAMsotvDimWwYAIq5bok="
    ),
    "d/8f2ed9d45ec81eba9c5612065ee66958": (
        "DNsg3pYBAAAAAAAAAAEotS/9YBUD1QsAhlJIOzClahuulzDl1gixOlxCrfnAEW9mlJEG5jesa6wdtjFTLXv/+FH4DQKbaozo4uuN"
        "ToZ2GN0xjSwjUrkDNgA0ADUAlNJpgWEYNlnbtdh7LXZrkOvRZbsWVOY8p2xFm3Y+2Z6/j70Sk3nNazLnnAZTk2iSK8uyjEoZYua5"
        "pLsHDL8OatLnfV1d/Fuf9P76nthTj9/7XoWfh71rXiKFoK+dy8HfR6BJBHqVpJNFA1tNkBJABYOy2vCLmcTDkOdrB8PJov71Gx4/"
        "1x4PO9fi3iYQv2fvL/T1MaHM49cllOh9ffsBLY4NQkYhZIBi40PzsKBqdUBoHAP3rc9IBmcJBKTs6uhwkeIKAlw0IHQzUkQCIq7H"
        "SCsOpOzGyoTGdRqYlF3dAiAgQAJjmAp4B6TcxgufZOGA5INFWiD4mToc8ygBa0MgtFHwdsMpnNhozOC/FyzoRuEWXIAF4AWGitrr"
        "Z6tEubgCmj2KuGtQiKWGomPWHR3f9Oxj1qC+K8QgPw=="
    ),
    "_METADATA": (
        "eyJ0cmVlX21ldGFkYXRhIjogeyIoJ3cxJywgJ2JpYXMnLCAndmFsdWUnKSI6IHsia2V5X21ldGFkYXRhIjogW3sia2V5IjogIncx"
        "IiwgImtleV90eXBlIjogMn0sIHsia2V5IjogImJpYXMiLCAia2V5X3R5cGUiOiAyfSwgeyJrZXkiOiAidmFsdWUiLCAia2V5X3R5"
        "cGUiOiAyfV0sICJ2YWx1ZV9tZXRhZGF0YSI6IHsidmFsdWVfdHlwZSI6ICJqYXguQXJyYXkiLCAic2tpcF9kZXNlcmlhbGl6ZSI6"
        "IGZhbHNlLCAid3JpdGVfc2hhcGUiOiBbMV19fSwgIigndzEnLCAna2VybmVsJywgJ3ZhbHVlJykiOiB7ImtleV9tZXRhZGF0YSI6"
        "IFt7ImtleSI6ICJ3MSIsICJrZXlfdHlwZSI6IDJ9LCB7ImtleSI6ICJrZXJuZWwiLCAia2V5X3R5cGUiOiAyfSwgeyJrZXkiOiAi"
        "dmFsdWUiLCAia2V5X3R5cGUiOiAyfV0sICJ2YWx1ZV9tZXRhZGF0YSI6IHsidmFsdWVfdHlwZSI6ICJqYXguQXJyYXkiLCAic2tp"
        "cF9kZXNlcmlhbGl6ZSI6IGZhbHNlLCAid3JpdGVfc2hhcGUiOiBbMSwgMl19fSwgIigndzInLCAnYmlhcycsICd2YWx1ZScpIjog"
        "eyJrZXlfbWV0YWRhdGEiOiBbeyJrZXkiOiAidzIiLCAia2V5X3R5cGUiOiAyfSwgeyJrZXkiOiAiYmlhcyIsICJrZXlfdHlwZSI6"
        "IDJ9LCB7ImtleSI6ICJ2YWx1ZSIsICJrZXlfdHlwZSI6IDJ9XSwgInZhbHVlX21ldGFkYXRhIjogeyJ2YWx1ZV90eXBlIjogImph"
        "eC5BcnJheSIsICJza2lwX2Rlc2VyaWFsaXplIjogZmFsc2UsICJ3cml0ZV9zaGFwZSI6IFsyXX19LCAiKCd3MicsICdrZXJuZWwn"
        "LCAndmFsdWUnKSI6IHsia2V5X21ldGFkYXRhIjogW3sia2V5IjogIncyIiwgImtleV90eXBlIjogMn0sIHsia2V5IjogImtlcm5l"
        "bCIsICJrZXlfdHlwZSI6IDJ9LCB7ImtleSI6ICJ2YWx1ZSIsICJrZXlfdHlwZSI6IDJ9XSwgInZhbHVlX21ldGFkYXRhIjogeyJ2"
        "YWx1ZV90eXBlIjogImpheC5BcnJheSIsICJza2lwX2Rlc2VyaWFsaXplIjogZmFsc2UsICJ3cml0ZV9zaGFwZSI6IFsyLCAxXX19"
        "fSwgInVzZV96YXJyMyI6IGZhbHNlLCAic3RvcmVfYXJyYXlfZGF0YV9lcXVhbF90b19maWxsX3ZhbHVlIjogdHJ1ZSwgImN1c3Rv"
        "bV9tZXRhZGF0YSI6IG51bGx9"
    ),
}


def _materialise(tmp_path):
  for rel, b64 in GOLDEN.items():
    p = tmp_path / rel
    p.parent.mkdir(parents=True, exist_ok=True)
    p.write_bytes(base64.b64decode(b64))
  return str(tmp_path)


def test_reads_an_orbax_written_checkpoint(tmp_path):
  d = _materialise(tmp_path)
  st = ocdbt.OcdbtStore(d)                      # verifies the crc32c of the manifest and of every node
  assert st.generation == 1 and len(st.keys()) == 17
  assert st.get("w1.kernel.value/.zarray").startswith(b'{"chunks":[1,2]')
  assert st.get("nope") is None
  tree = orbax_layout.read_tree(d)
  assert {k: tuple(v.shape) for k, v in tree.items()} == {
      ("w1", "bias", "value"): (4,), ("w1", "kernel", "value"): (2, 4),
      ("w2", "bias", "value"): (2,), ("w2", "kernel", "value"): (4, 2)}
  np.testing.assert_allclose(tree[("w1", "kernel", "value")].numpy()[0],
                             [0.7567299, -0.68570054, -0.5688337, -0.8757605], rtol=1e-6)
  assert not tree[("w1", "bias", "value")].any()


def test_corruption_is_detected(tmp_path):
  d = _materialise(tmp_path)
  p = tmp_path / "d" / "8f2ed9d45ec81eba9c5612065ee66958"
  raw = bytearray(p.read_bytes())
  raw[40] ^= 0xFF
  p.write_bytes(bytes(raw))
  with pytest.raises(ocdbt.OcdbtError, match="crc32c"):
    ocdbt.OcdbtStore(d).keys()
  with pytest.raises(ocdbt.OcdbtError, match="magic"):
    (tmp_path / "manifest.ocdbt").write_bytes(b"\x00" * 64)
    ocdbt.OcdbtStore(d)


@pytest.mark.parametrize("leaf_size", [0, 3])
def test_writer_round_trip_with_out_of_line_values_and_interior_nodes(tmp_path, leaf_size):
  rng = np.random.default_rng(0)
  items = {f"layer{i}.w.value/{j}.0": rng.bytes(300 + 17 * i + j) for i in range(4) for j in range(3)}
  items.update({f"layer{i}.w.value/.zarray": b'{"zarr_format":2}' for i in range(4)})
  ocdbt.write_store(str(tmp_path), items, max_inline=100, leaf_size=leaf_size)
  st = ocdbt.OcdbtStore(str(tmp_path))
  assert st.keys() == sorted(items)
  for k, v in items.items():
    assert st.get(k) == v, k
  assert ocdbt.crc32c(b"123456789") == 0xE3069283


def test_orbax_tree_in_an_ocdbt_container(tmp_path):
  """Our own zarr tree re-packed into an OCDBT store reads back through the same entry point."""
  tree = {("a", "w", "value"): torch.arange(12, dtype=torch.float32).view(3, 4),
          ("b", 0, "value"): torch.ones(5, dtype=torch.bfloat16)}
  plain = tmp_path / "plain"
  orbax_layout.write_tree(str(plain), tree)
  items = {}
  for root, _, files in os.walk(plain):
    for f in files:
      rel = os.path.relpath(os.path.join(root, f), plain)
      if rel.startswith(("_", "array_metadatas")):
        continue
      items[rel.replace(os.sep, "/")] = open(os.path.join(root, f), "rb").read()
  packed = tmp_path / "packed"
  packed.mkdir()
  for meta in ("_METADATA", "_sharding"):
    if (plain / meta).exists():
      (packed / meta).write_bytes((plain / meta).read_bytes())
  ocdbt.write_store(str(packed), items, max_inline=16)
  got = orbax_layout.read_tree(str(packed))
  assert set(got) == set(tree)
  for k in tree:
    assert torch.equal(got[k], tree[k])
