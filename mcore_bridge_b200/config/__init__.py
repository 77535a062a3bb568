from .model_config import ModelConfig
from .parser import hf_to_mcore_config
