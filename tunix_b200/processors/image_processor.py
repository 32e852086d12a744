"""Image preprocessing for vision-language models (tunix/processors/image_processor.py).

Two pipelines. `ImageProcessor` is the fixed-resolution one (Gemma 3 / SigLIP): bilinear resize
to (height, width), `(x - mean) / std`, clip to [-1, 1], zero images as padding up to the largest
image count in the batch. The functions below it are the variable-resolution pipeline
(Gemma 4): aspect-preserving bicubic resize so that the image tiles into at most
`max_soft_tokens * pool^2` patches with both sides multiples of `pool * patch`, patchify with
(x, y) patch positions, pad patches (positions -1), and expand each image placeholder token
of the prompt into `\\n\\n <start> soft*count <end> \\n\\n`.
"""
from __future__ import annotations

import math
from typing import Any, List, Optional, Sequence, Tuple, Union

import einops
import numpy as np
from PIL import Image

POSITIONS_PAD_VALUE = -1
SOFT_TOKEN_PLACEHOLDER = -2      # replaced by vision embeddings inside the model
DOUBLE_NEW_LINE_TOKEN = 108

ImageLike = Union[str, np.ndarray, "Image.Image", None]


def _per_sample_lists(images: Any) -> List[list]:
  """One image, one image per sample, or per-sample lists (None / [] = no image) -> a list of lists."""
  if not isinstance(images, list):
    return [[images]]
  return [[] if s is None else (list(s) if isinstance(s, (list, tuple)) else [s]) for s in images]


def _compute_max_num_images(lst) -> int:
  return max((len(s) for s in _per_sample_lists(lst)), default=0) if isinstance(lst, list) else 1


class ImageProcessor:
  """Fixed-resolution processor; `config` needs image_height/width/channels/mean/std. The batch is produced in one
  zero-filled [B, I, H, W, C] array (samples with fewer images keep zeros) and handed out as nested views."""

  def __init__(self, config: Any):
    self.config = config
    self._hwc = (config.image_height, config.image_width, config.image_channels)
    self._shift = np.asarray(config.image_mean, dtype=np.float32)
    self._scale = 1.0 / np.asarray(config.image_std, dtype=np.float32)

  def __call__(self, images) -> List[List[np.ndarray]]:
    samples = _per_sample_lists(images)
    slots = max((len(s) for s in samples), default=0)
    batch = np.zeros((len(samples), slots) + self._hwc, dtype=np.float32)
    for b, sample in enumerate(samples):
      for i, image in enumerate(sample):
        batch[b, i] = self.preprocess_image(image)
    return [[batch[b, i] for i in range(slots)] for b in range(len(samples))]

  def _open(self, image: ImageLike) -> "Image.Image":
    opened = Image.open(image) if isinstance(image, str) else \
        Image.fromarray(image) if isinstance(image, np.ndarray) else image
    return opened.convert("RGB") if self._hwc[2] == 3 else opened

  def preprocess_image(self, image: ImageLike) -> np.ndarray:
    """Bilinear resize, `(x - mean) / std`, clip to [-1, 1]; None gives the all-zero padding image."""
    height, width, channels = self._hwc
    if image is None:
      return np.zeros(self._hwc, dtype=np.float32)
    pixels = np.asarray(self._open(image).resize((width, height), resample=Image.Resampling.BILINEAR), dtype=np.float32)
    pixels = pixels.reshape(height, width, -1)
    return np.clip((pixels - self._shift) * self._scale, -1.0, 1.0)


def get_target_dimensions(height: int, width: int, patch_size: int = 16, max_patches: int = 10080,
                          pooling_kernel_size: int = 3) -> Tuple[int, int]:
  """Largest (h, w) with the image's aspect ratio, sides multiples of pool*patch, h*w <= max_patches*patch^2.
  Worked in units of pooled cells (one cell = pool*patch pixels a side); a side that would round to zero cells
  gets one, and the other then gets the integer aspect ratio, capped by the cell budget."""
  cell = pooling_kernel_size * patch_size
  if height * width == 0:
    return cell, cell
  budget = max_patches // pooling_kernel_size ** 2                  # cells
  shrink = math.sqrt(max_patches * patch_size ** 2 / (height * width))
  cells = [int(shrink * side // cell) for side in (height, width)]
  if not any(cells):
    cells = [1, 1]
  else:
    for thin, long in ((0, 1), (1, 0)):
      if cells[thin] == 0:
        sides = (height, width)
        cells[thin], cells[long] = 1, min(max(1, sides[long] // sides[thin]), budget)
  return cells[0] * cell, cells[1] * cell


def aspect_ratio_preserving_resize(image: np.ndarray, patch_size: int = 16, max_patches: int = 10080,
                                   pooling_kernel_size: int = 3) -> np.ndarray:
  target = get_target_dimensions(*image.shape[:2], patch_size, max_patches, pooling_kernel_size)
  if target == tuple(image.shape[:2]):
    return image
  return np.asarray(Image.fromarray(image).resize(target[::-1], resample=Image.BICUBIC))


def _to_rgb_uint8(image) -> np.ndarray:
  if isinstance(image, Image.Image):
    return np.asarray(image.convert("RGB"))
  planes = image[..., None] if image.ndim == 2 else image
  if planes.shape[-1] == 1:
    return np.repeat(planes, 3, axis=-1)
  return planes[..., :3]                                            # drops an alpha plane


def preprocess_single_image(image, patch_size: int = 16, max_soft_tokens: int = 1120,
                            pooling_kernel_size: int = 3) -> np.ndarray:
  resized = aspect_ratio_preserving_resize(_to_rgb_uint8(image), patch_size,
                                           max_soft_tokens * pooling_kernel_size ** 2, pooling_kernel_size)
  return np.float32(1.0 / 255.0) * resized.astype(np.float32)


def num_soft_tokens_for_image(image: np.ndarray, patch_size: int = 16, pooling_kernel_size: int = 3) -> int:
  grid = np.asarray(image.shape[:2]) // patch_size
  return int(grid.prod() // pooling_kernel_size ** 2)


def preprocess_images_list(images: Sequence[Any], patch_size: int = 16, max_soft_tokens: int = 1120,
                           pooling_kernel_size: int = 3) -> Tuple[List[np.ndarray], List[int]]:
  done = [preprocess_single_image(im, patch_size, max_soft_tokens, pooling_kernel_size) for im in images]
  return done, [num_soft_tokens_for_image(p, patch_size, pooling_kernel_size) for p in done]


def patchify(images: np.ndarray, patch_size: int) -> Tuple[np.ndarray, np.ndarray]:
  """[..., H, W, C] -> patches [..., h*w, patch*patch*C] (row-major over the grid) and their (x, y)."""
  rows, cols = images.shape[-3] // patch_size, images.shape[-2] // patch_size
  cropped = images[..., :rows * patch_size, :cols * patch_size, :]
  patches = einops.rearrange(cropped, "... (r p) (c q) ch -> ... (r c) (p q ch)", p=patch_size, q=patch_size)
  y, x = np.divmod(np.arange(rows * cols), cols)
  xy = np.broadcast_to(np.stack([x, y], axis=-1), images.shape[:-3] + (rows * cols, 2))
  return patches, xy


def patchify_and_pad(images: Sequence[np.ndarray], patch_size: int = 16, max_patches: Optional[int] = None,
                     max_soft_tokens: int = 1120, pooling_kernel_size: int = 3):
  """Every image patchified into one row of zero-initialised [n, max_patches, D] / position [n, max_patches, 2]
  arrays (unused slots keep position -1); also the real patch count per image."""
  budget = max_soft_tokens * pooling_kernel_size ** 2 if max_patches is None else max_patches
  cut = [patchify(im, patch_size) for im in images]
  used = [p.shape[0] for p, _ in cut]
  length = max([budget] + used)
  patches = np.zeros((len(cut), length, cut[0][0].shape[-1]), dtype=cut[0][0].dtype)
  positions = np.full((len(cut), length, 2), POSITIONS_PAD_VALUE, dtype=cut[0][1].dtype)
  for i, (p, xy) in enumerate(cut):
    patches[i, :used[i]], positions[i, :used[i]] = p, xy
  return patches, positions, used


def preprocess_and_patchify(images: Sequence[Any], patch_size: int = 16, max_soft_tokens: int = 1120,
                            pooling_kernel_size: int = 3):
  done, counts = preprocess_images_list(images, patch_size, max_soft_tokens, pooling_kernel_size)
  patches, xy, _ = patchify_and_pad(done, patch_size, None, max_soft_tokens, pooling_kernel_size)
  return patches, xy, counts


def _expand_row(row: np.ndarray, counts: Sequence[int], placeholder_token: int, start_token: int,
                end_token: int) -> np.ndarray:
  """Scatter form of the expansion: each token knows its output length (1, or count + 4 for the first
  len(counts) placeholders), the exclusive prefix sum gives its output offset."""
  row = np.asarray(row)
  holes = np.flatnonzero(row == placeholder_token)[:len(counts)]
  sizes = np.asarray(counts[:len(holes)], dtype=np.int64)
  span = np.ones(row.shape[0], dtype=np.int64)
  span[holes] = sizes + 4
  offset = np.cumsum(span) - span
  out = np.full(int(span.sum()), SOFT_TOKEN_PLACEHOLDER, dtype=np.int32)
  keep = np.ones(row.shape[0], dtype=bool)
  keep[holes] = False
  out[offset[keep]] = row[keep]
  first, last = offset[holes], offset[holes] + sizes + 3
  out[first], out[first + 1] = DOUBLE_NEW_LINE_TOKEN, start_token
  out[last - 1], out[last] = end_token, DOUBLE_NEW_LINE_TOKEN
  return out


def _right_pad(rows: Sequence[np.ndarray], fill: int, dtype) -> np.ndarray:
  out = np.full((len(rows), max(len(r) for r in rows)), fill, dtype=dtype)
  for b, r in enumerate(rows):
    out[b, :len(r)] = r
  return out


def add_variable_extra_tokens_for_images(tokens: np.ndarray, *, soft_token_counts, placeholder_token: int = 258880,
                                         start_token: int = 255999, end_token: int = 258882) -> np.ndarray:
  """Replaces the i-th placeholder of a row by `\\n\\n <start> soft*count_i <end> \\n\\n`; rows are
  right-padded with 0 to the longest result. `soft_token_counts` is one list for all rows or a
  tuple of per-row tuples."""
  shared = len(soft_token_counts) > 0 and np.isscalar(soft_token_counts[0])
  def counts_of(b):
    if shared:
      return list(soft_token_counts)
    return list(soft_token_counts[b]) if b < len(soft_token_counts) else []
  return _right_pad([_expand_row(tokens[b], counts_of(b), placeholder_token, start_token, end_token)
                     for b in range(tokens.shape[0])], 0, np.int32)


def process_gemma4_inputs(images: Any, tokens: List[np.ndarray], vision_encoder: Any, pad_id: int):
  """Per-sample image lists + token rows -> ((patches [B, I*P, D], positions [B, I*P, 2]) or None,
  expanded token rows). Samples with fewer images are padded with empty images (positions -1)."""
  vc = vision_encoder.config
  samples = _per_sample_lists(images)
  cut = [preprocess_and_patchify(s, vc.patch_size, vc.num_mm_tokens_per_image, vc.pooling_kernel_size) if s else None
         for s in samples]
  counts = [tuple(c[2]) if c else () for c in cut]
  expanded = [_expand_row(row, counts[b], 258880, 255999, 258882) for b, row in enumerate(tokens)]
  longest = max(len(r) for r in expanded)
  new_tokens = [np.concatenate([r.astype(np.asarray(tokens[b]).dtype),
                                np.full(longest - len(r), pad_id, np.asarray(tokens[b]).dtype)])
                for b, r in enumerate(expanded)]
  slots = max((len(s) for s in samples), default=0)
  if slots == 0:
    return None, new_tokens
  length = max(c[0].shape[1] for c in cut if c)
  patches = np.zeros((len(samples), slots, length, 3 * vc.patch_size ** 2), dtype=np.float32)
  positions = np.full((len(samples), slots, length, 2), POSITIONS_PAD_VALUE, dtype=np.int64)
  for b, c in enumerate(cut):
    if c:
      patches[b, :c[0].shape[0]], positions[b, :c[1].shape[0]] = c[0], c[1]
  return (patches.reshape(len(samples), slots * length, -1), positions.reshape(len(samples), slots * length, 2)), new_tokens
