"""Scaffolding for token-diffusion training objectives."""
from .types import DiffusionTokenBatch, validate_diffusion_logits
from .interfaces import DiffusionBatchAdapter, DiffusionLogitsFn, compute_diffusion_logits, masked_token_loss
