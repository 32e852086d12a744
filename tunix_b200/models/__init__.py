"""Model zoo: one decoder (`transformer.Transformer`) configured per family."""
from .transformer import AttentionType, ModelConfig, RematConfig, Transformer  # noqa: F401
