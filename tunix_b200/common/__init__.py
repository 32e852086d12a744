"""Configuration dataclasses and enums shared by every workflow."""
from .configs import CacheConfig, ClusterConfig, RLTrainingConfig, RolloutConfig, TrainingConfig  # noqa: F401
from .datatypes import Mode, Role  # noqa: F401
