"""Gemma 4 text decoder."""
from .model import AttentionType, Gemma4, ModelConfig, kv_sharing_pattern  # noqa: F401
