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

import numpy as np
from PIL import Image

POSITIONS_PAD_VALUE = -1
SOFT_TOKEN_PLACEHOLDER = -2      # replaced by vision embeddings inside the model
DOUBLE_NEW_LINE_TOKEN = 108

ImageLike = Union[str, np.ndarray, "Image.Image", None]


class ImageProcessor:
  """Fixed-resolution processor; `config` needs image_height/width/channels/mean/std."""

  def __init__(self, config: Any):
    self._height = config.image_height
    self._width = config.image_width
    self._channels = config.image_channels
    self._mean = np.asarray(config.image_mean, dtype=np.float32)
    self._std = np.asarray(config.image_std, dtype=np.float32)
    self.config = config

  def _blank(self) -> np.ndarray:
    return np.zeros((self._height, self._width, self._channels), dtype=np.float32)

  def __call__(self, images) -> List[List[np.ndarray]]:
    """A single image, a list with one image per sample, or a list of per-sample lists
    (None = a sample without images). Returns [batch][max images] arrays of [H, W, C] float32."""
    if not isinstance(images, list):
      images = [[images]]
    most = _compute_max_num_images(images)
    out = []
    for sample in images:
      if sample is None:
        items = []
      elif isinstance(sample, list):
        items = sample
      else:
        items = [sample]
      done = [self.preprocess_image(im) for im in items]
      done += [self._blank() for _ in range(most - len(done))]
      out.append(done)
    return out

  def preprocess_image(self, image: ImageLike) -> np.ndarray:
    if image is None:
      return self._blank()
    if isinstance(image, str):
      image = Image.open(image)
    elif isinstance(image, np.ndarray):
      image = Image.fromarray(image)
    if self._channels == 3:
      image = image.convert("RGB")
    image = image.resize((self._width, self._height), resample=Image.Resampling.BILINEAR)   # PIL: width first
    arr = np.array(image, dtype=np.float32)
    if arr.ndim == 2:
      arr = arr[..., None]
    return np.clip((arr - self._mean) / self._std, -1.0, 1.0)


def _compute_max_num_images(lst) -> int:
  best = 0
  for item in lst:
    if isinstance(item, list):
      best = max(best, len(item))
    elif item is not None:
      best = max(best, 1)
  return best


def get_target_dimensions(height: int, width: int, patch_size: int = 16, max_patches: int = 10080,
                          pooling_kernel_size: int = 3) -> Tuple[int, int]:
  """Largest (h, w) with the image's aspect ratio, sides multiples of pool*patch, h*w <= max_patches*patch^2."""
  side = pooling_kernel_size * patch_size
  if height * width == 0:
    return side, side
  f = math.sqrt(max_patches * patch_size ** 2 / (height * width))
  th = int(math.floor(f * height / side)) * side
  tw = int(math.floor(f * width / side)) * side
  longest = (max_patches // pooling_kernel_size ** 2) * side
  if th == 0 and tw == 0:
    th = tw = side
  elif th == 0:       # extremely wide: one row of pooled cells
    th = side
    tw = min(max(1, width // height) * side, longest)
  elif tw == 0:
    tw = side
    th = min(max(1, height // width) * side, longest)
  return int(th), int(tw)


def aspect_ratio_preserving_resize(image: np.ndarray, patch_size: int = 16, max_patches: int = 10080,
                                   pooling_kernel_size: int = 3) -> np.ndarray:
  h, w = image.shape[:2]
  th, tw = get_target_dimensions(h, w, patch_size, max_patches, pooling_kernel_size)
  if (th, tw) == (h, w):
    return image
  return np.array(Image.fromarray(image).resize((tw, th), resample=Image.BICUBIC))


def _to_rgb_uint8(image) -> np.ndarray:
  if isinstance(image, Image.Image):
    return np.array(image.convert("RGB"))
  if image.ndim == 2:
    return np.stack([image] * 3, axis=-1)
  if image.shape[-1] == 4:
    return image[..., :3]
  if image.shape[-1] == 1:
    return np.concatenate([image] * 3, axis=-1)
  return image


def preprocess_single_image(image, patch_size: int = 16, max_soft_tokens: int = 1120,
                            pooling_kernel_size: int = 3) -> np.ndarray:
  image = _to_rgb_uint8(image)
  image = aspect_ratio_preserving_resize(image, patch_size, max_soft_tokens * pooling_kernel_size ** 2,
                                         pooling_kernel_size)
  return image.astype(np.float32) / 255.0


def num_soft_tokens_for_image(image: np.ndarray, patch_size: int = 16, pooling_kernel_size: int = 3) -> int:
  h, w = image.shape[:2]
  return int((h // patch_size) * (w // patch_size) // pooling_kernel_size ** 2)


def preprocess_images_list(images: Sequence[Any], patch_size: int = 16, max_soft_tokens: int = 1120,
                           pooling_kernel_size: int = 3) -> Tuple[List[np.ndarray], List[int]]:
  done = [preprocess_single_image(im, patch_size, max_soft_tokens, pooling_kernel_size) for im in images]
  return done, [num_soft_tokens_for_image(p, patch_size, pooling_kernel_size) for p in done]


def patchify(images: np.ndarray, patch_size: int) -> Tuple[np.ndarray, np.ndarray]:
  """[..., H, W, C] -> patches [..., h*w, patch*patch*C] (row-major over the grid) and their (x, y)."""
  *lead, H, W, C = images.shape
  h, w = H // patch_size, W // patch_size
  x = images[..., :h * patch_size, :w * patch_size, :].reshape(*lead, h, patch_size, w, patch_size, C)
  n = len(lead)
  x = np.transpose(x, list(range(n)) + [n, n + 2, n + 1, n + 3, n + 4])
  patches = x.reshape(*lead, h * w, patch_size * patch_size * C)
  gx, gy = np.meshgrid(np.arange(w), np.arange(h))
  pos = np.stack([gx, gy], axis=-1).reshape(h * w, 2)
  return patches, np.broadcast_to(pos, tuple(lead) + (h * w, 2))


def patchify_and_pad(images: Sequence[np.ndarray], patch_size: int = 16, max_patches: Optional[int] = None,
                     max_soft_tokens: int = 1120, pooling_kernel_size: int = 3):
  if max_patches is None:
    max_patches = max_soft_tokens * pooling_kernel_size ** 2
  P, XY, real = [], [], []
  for im in images:
    p, xy = patchify(im[None], patch_size)
    p, xy = p[0], xy[0]
    real.append(p.shape[0])
    pad = max_patches - p.shape[0]
    if pad > 0:
      p = np.concatenate([p, np.zeros((pad, p.shape[-1]), p.dtype)], axis=0)
      xy = np.concatenate([xy, np.full((pad, 2), POSITIONS_PAD_VALUE, xy.dtype)], axis=0)
    P.append(p)
    XY.append(xy)
  return np.stack(P, 0), np.stack(XY, 0), real


def preprocess_and_patchify(images: Sequence[Any], patch_size: int = 16, max_soft_tokens: int = 1120,
                            pooling_kernel_size: int = 3):
  done, counts = preprocess_images_list(images, patch_size, max_soft_tokens, pooling_kernel_size)
  patches, xy, _ = patchify_and_pad(done, patch_size, None, max_soft_tokens, pooling_kernel_size)
  return patches, xy, counts


def add_variable_extra_tokens_for_images(tokens: np.ndarray, *, soft_token_counts, placeholder_token: int = 258880,
                                         start_token: int = 255999, end_token: int = 258882) -> np.ndarray:
  """Replaces the i-th placeholder of a row by `\\n\\n <start> soft*count_i <end> \\n\\n`; rows are
  right-padded with 0 to the longest result. `soft_token_counts` is one list for all rows or a
  tuple of per-row tuples."""
  rows = []
  flat = len(soft_token_counts) > 0 and isinstance(soft_token_counts[0], (int, np.integer))
  for b in range(tokens.shape[0]):
    counts = soft_token_counts if flat else (soft_token_counts[b] if b < len(soft_token_counts) else ())
    out, k = [], 0
    for t in tokens[b].tolist():
      if t == placeholder_token and k < len(counts):
        out += [DOUBLE_NEW_LINE_TOKEN, start_token] + [SOFT_TOKEN_PLACEHOLDER] * int(counts[k]) + \
            [end_token, DOUBLE_NEW_LINE_TOKEN]
        k += 1
      else:
        out.append(t)
    rows.append(out)
  width = max(len(r) for r in rows)
  padded = np.zeros((len(rows), width), dtype=np.int32)
  for b, r in enumerate(rows):
    padded[b, :len(r)] = r
  return padded


def process_gemma4_inputs(images: Any, tokens: List[np.ndarray], vision_encoder: Any, pad_id: int):
  """Per-sample image lists + token rows -> ((patches [B, I*P, D], positions [B, I*P, 2]) or None,
  expanded token rows). Samples with fewer images are padded with empty images (positions -1)."""
  if not isinstance(images, list):
    images = [[images]]
  elif images and not isinstance(images[0], list):
    images = [[im] for im in images]
  vc = vision_encoder.config
  most = max((len(s) for s in images), default=0)
  per_sample, counts_all, width = [], [], 0
  for sample in images:
    if not sample:
      per_sample.append(None)
      counts_all.append(())
      continue
    p, xy, counts = preprocess_and_patchify(sample, vc.patch_size, vc.num_mm_tokens_per_image,
                                            vc.pooling_kernel_size)
    per_sample.append((p, xy))
    counts_all.append(tuple(counts))
    width = max(width, p.shape[1])
  if width == 0:
    width = vc.num_mm_tokens_per_image * vc.pooling_kernel_size ** 2
  dim = 3 * vc.patch_size ** 2
  P, XY = [], []
  for item in per_sample:
    if item is None:
      p = np.zeros((0, width, dim), np.float32)
      xy = np.full((0, width, 2), POSITIONS_PAD_VALUE, np.int64)
    else:
      p, xy = item
    pad = most - p.shape[0]
    if pad > 0:
      p = np.concatenate([p, np.zeros((pad, width, dim), p.dtype)], 0)
      xy = np.concatenate([xy, np.full((pad, width, 2), POSITIONS_PAD_VALUE, xy.dtype)], 0)
    P.append(p.reshape(most * width, dim))
    XY.append(xy.reshape(most * width, 2))
  new_tokens = []
  for b, row in enumerate(tokens):
    row = np.asarray(row)[None]
    new_tokens.append(add_variable_extra_tokens_for_images(row, soft_token_counts=(counts_all[b],))[0])
  width_t = max(len(r) for r in new_tokens)
  new_tokens = [np.concatenate([r, np.full(width_t - len(r), pad_id, r.dtype)]) for r in new_tokens]
  if most == 0:
    return None, new_tokens
  return (np.stack(P, 0), np.stack(XY, 0)), new_tokens
