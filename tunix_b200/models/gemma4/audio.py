"""Gemma 4 audio tower (tunix/models/gemma4/audio.py:33-1248): log-mel front end, 4x convolutional subsampling and
a stack of streaming Conformer layers that turn a 16 kHz waveform into soft tokens for the decoder.

Pipeline for waveforms [B, samples] with true lengths [B]:

  mel          frames of 320 samples every 160 (a 321-sample unfold with the last sample dropped), a Hann window
               that never touches zero, 512-point rFFT magnitude, 128 HTK-mel triangles, log(x + 1e-3);
  subsampling  two 3 x 3 stride-2 convolutions over (time, mel) with channel LayerNorm + ReLU, then a linear map of
               the (mel / 4) x 32 remaining features to the model width; the validity mask is thinned alongside;
  conformer    per layer: half-step FFN, local self-attention, causal depthwise convolution (GLU in, SiLU out),
               half-step FFN, RMS norm - every residual branch wrapped in value clamps;
  output       linear map to `lm_model_dims`, padding frames zeroed.

Attention is written as what it is - a *band*: frame t attends frames t - (left_context - 1) .. t + right_context
that are valid - instead of the reference's blocks of 12 queries with a relative-shift trick. For every offset j
of the band, logit = q_t . k_{t-L+j} + q_t . E_j, where E_j is a learned projection of the sinusoidal embedding of
the distance L - j (Transformer-XL style); logits are soft-capped at 50, masked to -1e9 and soft-maxed over the
band. The band form needs one [B, T, heads, band] tensor instead of five-dimensional block tensors and gives
identical numbers, since blocks only ever tile this band.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional, Tuple

import numpy as np
import torch
from torch import nn

from ...ops import functional as F

_EPS = 1e-6
_SOFTCAP = 50.0
_R_SOFTPLUS_0 = 1.442695041            # 1 / softplus(0)
_MASKED = -1e9


@dataclasses.dataclass
class ConformerConfig:
  num_layers: int = 12
  model_dims: int = 1024
  lm_model_dims: int = 1536
  atten_num_heads: int = 8
  atten_left_context: int = 13
  atten_right_context: int = 0
  atten_block_size: int = 12           # block size of the reference's formulation; the band does not depend on it
  conv_kernel_size: int = 5
  gradient_clipping: float = 10_000_000_000.0
  conf_reduction_factor: int = 1


# ------------------------------------------------------------------------------------------ mel front end
class MelFilterbank:
  """Log-mel spectrogram with fixed tables (no parameters)."""

  def __init__(self, sample_rate: int = 16000, win_length: int = 320, hop_length: int = 160, n_mels: int = 128,
               f_min: float = 0.0, f_max: float = 8000.0, constant: float = 1e-3):
    self.sample_rate, self.win_length, self.hop_length, self.n_mels = sample_rate, win_length, hop_length, n_mels
    self.constant = constant
    self.n_fft = 1 << int(math.ceil(math.log2(win_length)))
    n = np.arange(win_length, dtype=np.float32)
    self.window = torch.from_numpy(0.5 - 0.5 * np.cos(2.0 * np.pi / win_length * (n + 0.5))).float()
    self.mel_basis = torch.from_numpy(self._triangles(f_min, f_max)).float()          # [n_fft / 2 + 1, n_mels]

  def _triangles(self, f_min: float, f_max: float) -> np.ndarray:
    to_mel = lambda hz: 2595.0 * np.log10(1.0 + hz / 700.0)
    to_hz = lambda mel: 700.0 * (np.power(10.0, mel / 2595.0) - 1.0)
    bins = np.linspace(0.0, self.sample_rate / 2.0, self.n_fft // 2 + 1, dtype=np.float64)
    edges = to_hz(np.linspace(to_mel(f_min), to_mel(f_max), self.n_mels + 2))
    width = np.diff(edges)
    rel = edges[None, :] - bins[:, None]
    rising = -rel[:, :-2] / width[:-1]
    falling = rel[:, 2:] / width[1:]
    return np.maximum(0.0, np.minimum(rising, falling)).astype(np.float32)

  def num_frames(self, num_samples: int) -> int:
    span = self.win_length + 1
    return 0 if num_samples < span else (num_samples - span) // self.hop_length + 1

  def __call__(self, waveform: torch.Tensor) -> torch.Tensor:
    """[B, samples] -> [B, frames, n_mels]."""
    frames = waveform.unfold(-1, self.win_length + 1, self.hop_length)[..., :-1]
    spec = torch.fft.rfft(frames * self.window.to(waveform.device), n=self.n_fft).abs()
    return torch.log(spec @ self.mel_basis.to(waveform.device) + self.constant)


def to_float32(x: torch.Tensor) -> torch.Tensor:
  """PCM integers to [-1, 1) floats; floats pass through."""
  if x.dtype == torch.int16:
    return x.float() / 32768.0
  if x.dtype == torch.int32:
    return x.float() / 2147483648.0
  if x.dtype == torch.uint8:
    return (x.float() - 128.0) / 128.0
  if x.dtype in (torch.float16, torch.float32, torch.bfloat16):
    return x.float()
  raise ValueError(f"Unsupported format: {x.dtype}")


# ------------------------------------------------------------------------------------------ building blocks
def _rms(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
  xf = x.float()
  return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + _EPS) * scale.float()).to(x.dtype)


class _Clipped(nn.Module):
  """Linear map with checkpoint-provided clamps on its input and output (infinite = off)."""

  def __init__(self, out_features: int, in_features: int, dtype, device=None):
    super().__init__()
    self.w = nn.Parameter(torch.zeros(out_features, in_features, dtype=dtype, device=device))
    for name, value in (("clip_input_min", -math.inf), ("clip_input_max", math.inf),
                        ("clip_output_min", -math.inf), ("clip_output_max", math.inf)):
      self.register_buffer(name, torch.tensor(value, dtype=torch.float32, device=device))

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    x = torch.clamp(x, self.clip_input_min.to(x.dtype), self.clip_input_max.to(x.dtype))
    y = F.linear(x.to(self.w.dtype), self.w)
    return torch.clamp(y, self.clip_output_min.to(y.dtype), self.clip_output_max.to(y.dtype))


class SubSampling(nn.Module):
  """[B, T, mel] -> [B, ~T / 4, D] and the thinned mask."""

  def __init__(self, in_features: int, out_features: int, dtype, device=None):
    super().__init__()
    kw = dict(dtype=dtype, device=device)
    self.conv0 = nn.Parameter(torch.zeros(128, 1, 3, 3, **kw))
    self.norm0 = nn.Parameter(torch.ones(128, **kw))
    self.conv1 = nn.Parameter(torch.zeros(32, 128, 3, 3, **kw))
    self.norm1 = nn.Parameter(torch.ones(32, **kw))
    self.input_proj = nn.Parameter(torch.zeros(out_features, (in_features // 4) * 32, **kw))

  @staticmethod
  def _stage(x, weight, norm_scale):
    x = torch.nn.functional.conv2d(x, weight, stride=2, padding=1)                    # [B, C, T', F']
    x = x.permute(0, 2, 3, 1)
    x = torch.nn.functional.layer_norm(x.float(), x.shape[-1:], norm_scale.float(), None, _EPS).to(x.dtype)
    return torch.relu(x).permute(0, 3, 1, 2)

  def forward(self, x: torch.Tensor, mask: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    x = x.to(self.conv0.dtype)[:, None]                                               # [B, 1, T, F]
    for weight, scale in ((self.conv0, self.norm0), (self.conv1, self.norm1)):
      x = self._stage(x, weight, scale)
      mask = mask[:, ::2][:, :x.shape[2]]
    B, C, T, Fm = x.shape
    feats = x.permute(0, 2, 3, 1).reshape(B, T, Fm * C)                               # (mel, channel) flattened
    return F.linear(feats, self.input_proj), mask


class FFN(nn.Module):
  """x + 0.5 * norm(W2 silu(W1 norm(x))), with value clamps around the branch."""

  def __init__(self, D: int, clip: float, dtype, device=None):
    super().__init__()
    self.clip = clip
    self.pre_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
    self.post_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
    self.up = _Clipped(4 * D, D, dtype, device)
    self.down = _Clipped(D, 4 * D, dtype, device)

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    y = self.down(torch.nn.functional.silu(self.up(_rms(x.clamp(-self.clip, self.clip), self.pre_norm))))
    return x + 0.5 * _rms(y.clamp(-self.clip, self.clip), self.post_norm)


class LightConv(nn.Module):
  """x + W_out silu(norm(causal depthwise conv(glu(W_in norm(x)))))."""

  def __init__(self, D: int, kernel: int, clip: float, dtype, device=None):
    super().__init__()
    self.clip, self.kernel = clip, kernel
    self.pre_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
    self.conv_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
    self.linear_start = _Clipped(2 * D, D, dtype, device)
    self.depthwise = nn.Parameter(torch.zeros(D, 1, kernel, dtype=dtype, device=device))
    self.linear_end = _Clipped(D, D, dtype, device)

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    y = torch.nn.functional.glu(self.linear_start(_rms(x, self.pre_norm)), dim=-1)
    y = torch.nn.functional.pad(y.transpose(1, 2), (self.kernel - 1, 0))              # frames see the past only
    y = torch.nn.functional.conv1d(y, self.depthwise, groups=y.shape[1]).transpose(1, 2)
    y = torch.nn.functional.silu(_rms(y.clamp(-self.clip, self.clip), self.conv_norm))
    return x + self.linear_end(y)


def sinusoid(distances: torch.Tensor, channels: int) -> torch.Tensor:
  """[n] distances -> [n, channels]: sines then cosines over timescales 1 .. 10^4 (geometric)."""
  half = channels // 2
  step = math.log(1.0e4) / max(half - 1, 1)
  inv = torch.exp(torch.arange(half, dtype=torch.float32, device=distances.device) * -step)
  angle = distances.float()[:, None] * inv[None, :]
  emb = torch.cat((angle.sin(), angle.cos()), dim=-1)
  return torch.nn.functional.pad(emb, (0, channels % 2))


class BandAttention(nn.Module):
  """Local self-attention over the band [t - L, t + R] with relative-position logits."""

  def __init__(self, cfg: ConformerConfig, dtype, device=None):
    super().__init__()
    D, self.N = cfg.model_dims, cfg.atten_num_heads
    self.H = D // self.N
    self.L, self.R = max(0, cfg.atten_left_context - 1), cfg.atten_right_context
    self.qkv = nn.ModuleList([_Clipped(D, D, dtype, device) for _ in range(3)])
    self.per_dim_scale = nn.Parameter(torch.ones(self.H, dtype=dtype, device=device))
    self.pos_proj = nn.Parameter(torch.zeros(D, D, dtype=dtype, device=device))       # [N H, channels]

  def _window(self, x: torch.Tensor, fill) -> torch.Tensor:
    """[B, T, ...] -> [B, T, band, ...]: entry j of frame t is frame t - L + j (fill outside the sequence)."""
    pad = [0, 0] * (x.dim() - 2) + [self.L, self.R]
    if x.dtype == torch.bool:
      padded = torch.nn.functional.pad(x.to(torch.uint8), pad, value=int(fill)).bool()
    else:
      padded = torch.nn.functional.pad(x, pad, value=fill)
    win = padded.unfold(1, self.L + self.R + 1, 1)                                    # [B, T, ..., band]
    return win.movedim(-1, 2)

  def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    B, T, _ = x.shape
    q, k, v = (proj(x).float().view(B, T, self.N, self.H) for proj in self.qkv)
    q = q * (_R_SOFTPLUS_0 / math.sqrt(self.H)) * torch.nn.functional.softplus(self.per_dim_scale.float())
    k = k * (_R_SOFTPLUS_0 * math.log1p(math.e))                                      # softplus(1)
    band = self.L + self.R + 1
    content = torch.einsum("btnh,btjnh->btnj", q, self._window(k, 0.0))
    distance = torch.arange(self.L, -self.R - 1, -1, device=x.device)                  # entry j <-> distance L - j
    E = F.linear(sinusoid(distance, self.N * self.H).to(self.pos_proj.dtype), self.pos_proj).float()
    position = torch.einsum("btnh,jnh->btnj", q, E.view(band, self.N, self.H))
    logits = _SOFTCAP * torch.tanh((content + position) / _SOFTCAP)
    visible = self._window(mask, False)                                               # [B, T, band]
    logits = torch.where(visible[:, :, None, :], logits, torch.full_like(logits, _MASKED))
    probs = torch.softmax(logits, dim=-1)
    return torch.einsum("btnj,btjnh->btnh", probs, self._window(v, 0.0))              # fp32 [B, T, N, H]


class ConformerLayer(nn.Module):

  def __init__(self, cfg: ConformerConfig, dtype, device=None):
    super().__init__()
    D, clip = cfg.model_dims, cfg.gradient_clipping
    self.clip = clip
    self.ffn_start = FFN(D, clip, dtype, device)
    self.attn_pre_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
    self.attn = BandAttention(cfg, dtype, device)
    self.attn_out = _Clipped(D, D, dtype, device)
    self.attn_post_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))
    self.lconv = LightConv(D, cfg.conv_kernel_size, clip, dtype, device)
    self.ffn_end = FFN(D, clip, dtype, device)
    self.final_norm = nn.Parameter(torch.ones(D, dtype=dtype, device=device))

  def forward(self, x: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    x = self.ffn_start(x)
    heads = self.attn(_rms(x.clamp(-self.clip, self.clip), self.attn_pre_norm), mask)
    y = self.attn_out(heads.reshape(*heads.shape[:2], -1).to(x.dtype))
    x = x + _rms(y.clamp(-self.clip, self.clip), self.attn_post_norm)
    x = x * mask[:, :, None].to(x.dtype)                     # the convolution must not smear padding into speech
    x = self.ffn_end(self.lconv(x))
    return _rms(x.clamp(-self.clip, self.clip), self.final_norm)


class AudioTokenizer(nn.Module):
  """`(waveforms [B, samples], lengths [B]) -> (soft tokens [B, T', lm_model_dims], padding mask [B, T'])`."""

  def __init__(self, config: ConformerConfig, dtype=torch.float32, device=None):
    super().__init__()
    self.config = config
    self.sample_rate = 16_000
    self.to_mel = MelFilterbank(sample_rate=self.sample_rate, n_mels=128)
    self.feature = SubSampling(128, config.model_dims, dtype, device)
    self.conformer_layers = nn.ModuleList([ConformerLayer(config, dtype, device) for _ in range(config.num_layers)])
    self.output_w = nn.Parameter(torch.zeros(config.lm_model_dims, config.model_dims, dtype=dtype, device=device))
    self.output_b = nn.Parameter(torch.zeros(config.lm_model_dims, dtype=dtype, device=device))

  def init_weights(self, seed: int = 0, scale: float = 0.02) -> "AudioTokenizer":
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
      for p in self.parameters():
        if p.dim() >= 2:
          p.copy_((torch.randn(p.shape, generator=g) * scale).to(p.dtype))
    return self

  @staticmethod
  def infer_mask(frames: int, sequence_lengths: torch.Tensor, original_len: int) -> torch.Tensor:
    """Validity of each of `frames` compressed steps given the true sample counts."""
    rate = original_len / frames
    valid = torch.floor(sequence_lengths.float() / rate).to(torch.int64)
    return torch.arange(frames, device=sequence_lengths.device)[None, :] < valid[:, None]

  def forward(self, x: torch.Tensor, sequence_lengths: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    x = to_float32(x)
    mel = self.to_mel(x)
    mask = self.infer_mask(mel.shape[1], sequence_lengths, x.shape[-1])
    h, mask = self.feature(torch.where(mask[:, :, None], mel, torch.zeros_like(mel)), mask)
    for layer in self.conformer_layers:
      h = layer(h, mask)
    stride = self.config.conf_reduction_factor
    if stride > 1:
      h, mask = h[:, ::stride], mask[:, ::stride]
    out = F.linear(h, self.output_w) + self.output_b
    return torch.where(mask[:, :, None], out, torch.zeros_like(out)), ~mask

  def get_num_soft_tokens(self, num_samples: int) -> int:
    frames = self.to_mel.num_frames(num_samples)
    if frames == 0:
      return 0
    for _ in range(2):                                   # two stride-2, kernel-3, padding-1 convolutions
      frames = (frames + 2 - 3) // 2 + 1
    return math.ceil(frames / self.config.conf_reduction_factor)


# ------------------------------------------------------------------------------------------ model-side glue
@dataclasses.dataclass
class PreprocessedAudioInput:
  """audios [B, clips, samples] (zero-padded) and sequence_lengths [B, clips] (true sample counts)."""
  audios: torch.Tensor
  sequence_lengths: torch.Tensor


def soft_tokens_per_row(encoder: AudioTokenizer, audio_input: PreprocessedAudioInput) -> Optional[torch.Tensor]:
  """Encodes every clip and packs each row's valid soft tokens to the front, clip after clip: [B, clips * T', D]
  with the padding frames (zeros) moved to the end, so the n-th audio placeholder of a row takes the n-th token."""
  B, clips = audio_input.audios.shape[:2]
  if clips == 0:
    return None
  emb, pad = encoder(audio_input.audios.reshape(B * clips, -1), audio_input.sequence_lengths.reshape(B * clips))
  emb, pad = emb.reshape(B, -1, emb.shape[-1]), pad.reshape(B, -1)
  order = torch.argsort(pad.to(torch.int8), dim=1, stable=True)                      # valid first, order kept
  return torch.gather(emb, 1, order[..., None].expand_as(emb))
