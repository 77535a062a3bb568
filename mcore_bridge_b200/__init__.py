"""B200-native model-definition and training framework with the public API of mcore-bridge.

Names are resolved lazily so ``import mcore_bridge_b200`` stays cheap (parity: reference
``src/mcore_bridge/__init__.py:18-33``).
"""
from typing import TYPE_CHECKING

if TYPE_CHECKING:
    from .bridge import GPTBridge
    from .config import ModelConfig, hf_to_mcore_config
    from .models import get_mcore_model
    from .tuners import LoraParallelLinear
    from .utils import get_logger, set_random_seed, split_cp_inputs, unwrap_model
    from .version import __release_datetime__, __version__
else:
    _import_structure = {
        'bridge': ['GPTBridge'],
        'config': ['ModelConfig', 'hf_to_mcore_config'],
        'models': ['get_mcore_model'],
        'tuners': ['LoraParallelLinear'],
        'utils': ['get_logger', 'set_random_seed', 'split_cp_inputs', 'unwrap_model'],
        'parallel': ['initialize_model_parallel', 'destroy_model_parallel'],
        'version': ['__release_datetime__', '__version__'],
    }
    from .utils.import_utils import lazy_exports
    __getattr__, __dir__, __all__ = lazy_exports(__name__, _import_structure)
