from .attention import AttentionProjectionStrategy, AttentionTransferStrategy
from .base_strategy import BaseStrategy, softmax_cross_entropy
from .feature_pooling import FeaturePoolingStrategy
from .feature_projection import FeatureProjectionStrategy
from .logit import LogitStrategy
