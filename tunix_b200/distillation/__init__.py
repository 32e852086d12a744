from . import feature_extraction, strategies
from .distillation_trainer import DistillationTrainer, TrainingInput
