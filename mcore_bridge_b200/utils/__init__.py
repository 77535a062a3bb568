from .dequantizer import Fp8Dequantizer, MxFp4Dequantizer, PackedDequantizer, fp4_to_fp8, quantize_fp8_blockwise
from .env import get_dist_setting, get_node_setting, is_dist, is_last_rank, is_local_master, is_master
from .import_utils import is_flash_attn_3_available, lazy_exports
from .logger import get_logger
from .safetensors import LazyTensor, SafetensorLazyLoader, StreamingSafetensorSaver
from .torch_utils import gc_collect, get_current_device, safe_ddp_context, to_device
from .utils import deep_getattr, get_env_args, json_parse_to_dict, patch_deepcopy
from .megatron_utils import (get_local_layer_specs, reconstruct_tensor_cp, roll_tensor, set_random_seed,  # noqa: E402
                             split_cp_inputs, unwrap_model)
