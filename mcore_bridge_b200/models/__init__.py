from .constant import LLMModelType, MLLMModelType, ModelType
from .register import (MODEL_MAPPING, ModelLoader, ModelMeta, get_mcore_model, get_mcore_model_type, get_model_meta,
                       register_model)
