from . import mappings, state  # noqa: F401
from .state import (destroy_model_parallel, get_state, init_distributed, initialize_model_parallel,  # noqa: F401
                    model_parallel_is_initialized)
