"""B200-native model-definition and training framework with the public API of mcore-bridge.

Names are resolved lazily so ``import mcore_bridge_b200`` stays cheap (parity: reference
``src/mcore_bridge/__init__.py:18-33``).
"""
import sys
from typing import TYPE_CHECKING

from .utils.import_utils import _LazyModule

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
    sys.modules[__name__] = _LazyModule(__name__, globals()['__file__'], _import_structure, module_spec=__spec__,
                                        extra_objects={})
