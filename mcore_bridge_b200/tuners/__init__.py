from .lora import LoraParallelLinear
from .patcher import apply_patch
from .peft_model import LoraConfig, LoraModel, ModulesToSaveWrapper, PeftModel, get_peft_model
from .utils import tuners_sharded_state_dict

apply_patch()
