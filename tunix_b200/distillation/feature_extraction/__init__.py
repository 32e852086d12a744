from .pooling import PaddingMode, avg_pool_array_to_target_shape
from .projection import (ModelWithFeatureProjection, remove_feature_projection_from_models,
                         setup_models_with_feature_projection)
from .sowed_module import (pop_sowed_intermediate_outputs, stack_features, unwrap_sowed_modules,
                           wrap_model_with_sowed_modules)
