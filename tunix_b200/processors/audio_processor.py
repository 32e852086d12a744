"""Audio preprocessing for Gemma4-E2B/E4B style decoders (tunix/processors/audio_processor.py).

Waveforms are grouped per sample (`[a1, [a2, a3], []]` = 1, 2 and 0 clips), padded to a common
length and clip count (fix both to keep shapes static across calls), and every audio placeholder
token of a prompt is expanded into `<start> soft*count <end>` where `count` comes from the
audio tokenizer for that clip's length.
"""
from __future__ import annotations

import dataclasses
from typing import List, Optional, Protocol, Sequence, Tuple, Union

import numpy as np

AUDIO_PLACEHOLDER_TOKEN = 258881
AUDIO_START_TOKEN = 256000
AUDIO_END_TOKEN = 258883
AUDIO_SOFT_TOKEN_PLACEHOLDER = -4
MAX_CLIP_SECONDS = 30


class AudioTokenizerLike(Protocol):
  sample_rate: int

  def get_num_soft_tokens(self, num_samples: int) -> int:
    ...


@dataclasses.dataclass
class PreprocessedAudioInput:
  waveforms: np.ndarray          # [B, clips, samples] float32, zero padded
  lengths: np.ndarray            # [B, clips] int32 true sample counts (0 = padding clip)
  soft_token_counts: Tuple[Tuple[int, ...], ...]


def _normalise(audios) -> List[List[np.ndarray]]:
  if isinstance(audios, np.ndarray):
    if audios.ndim != 1:
      raise ValueError("a single waveform must be one-dimensional")
    return [[audios]]
  if not isinstance(audios, list):
    raise ValueError(f"Unsupported audio waveform type {type(audios)}")
  out = []
  for clips in audios:
    if isinstance(clips, np.ndarray):
      clips = [clips]
    elif not isinstance(clips, list):
      raise ValueError(f"Unsupported audio waveform type {type(clips)}")
    if any(not isinstance(c, np.ndarray) or c.ndim != 1 for c in clips):
      raise ValueError("every clip must be a one-dimensional array")
    out.append(clips)
  return out


def expand_audio_tokens(row: Sequence[int], counts: Sequence[int]) -> np.ndarray:
  out, k = [], 0
  for t in list(row):
    if t == AUDIO_PLACEHOLDER_TOKEN and k < len(counts):
      out += [AUDIO_START_TOKEN] + [AUDIO_SOFT_TOKEN_PLACEHOLDER] * int(counts[k]) + [AUDIO_END_TOKEN]
      k += 1
    else:
      out.append(int(t))
  if k != len(counts):
    raise ValueError(f"prompt has {k} audio placeholders but {len(counts)} clips were given")
  return np.asarray(out, dtype=np.int32)


def process_gemma4_inputs(audios, tokens: List[np.ndarray], audio_encoder: AudioTokenizerLike,
                          max_audio_length: Optional[int] = None, max_audio_clips: Optional[int] = None):
  limit = audio_encoder.sample_rate * MAX_CLIP_SECONDS
  if max_audio_length is not None and max_audio_length > limit:
    raise ValueError(f"max_audio_length={max_audio_length} too big. Gemma4 supports maximum audio clip length of "
                     f"{limit} samples.")
  audios = _normalise(audios)
  if len(audios) != len(tokens):
    raise ValueError(f"Batch size of tokens ({len(tokens)}) does not match the batch size of audios "
                     f"({len(audios)}).")
  most_clips = max((len(c) for c in audios), default=0)
  if max_audio_clips is None:
    max_audio_clips = most_clips
  elif most_clips > max_audio_clips:
    raise ValueError(f'A batch entry has more clips than the specified "max_audio_clips". '
                     f"max_audio_clips={max_audio_clips}, actual_max_audio_clips={most_clips}.")
  longest = max((len(c) for clips in audios for c in clips), default=0)
  if longest > limit:
    raise ValueError(f"an audio clip has {longest} samples; the maximum is {limit}")
  if max_audio_length is None:
    max_audio_length = longest
  elif longest > max_audio_length:
    raise ValueError(f"an audio clip has {longest} samples but max_audio_length={max_audio_length}")
  counts = tuple(tuple(audio_encoder.get_num_soft_tokens(len(c)) for c in clips) for clips in audios)
  new_tokens = [expand_audio_tokens(np.asarray(row), counts[b]) for b, row in enumerate(tokens)]
  if most_clips == 0 and max_audio_clips == 0:
    return None, new_tokens
  wave = np.zeros((len(audios), max_audio_clips, max_audio_length), np.float32)
  lens = np.zeros((len(audios), max_audio_clips), np.int32)
  for b, clips in enumerate(audios):
    for i, c in enumerate(clips):
      wave[b, i, :len(c)] = c
      lens[b, i] = len(c)
  return PreprocessedAudioInput(wave, lens, counts), new_tokens
