"""Qwen3-Next: hybrid stack of gated-DeltaNet linear-attention layers and gated full-attention layers, MoE with a
gated shared expert, zero-centred RMSNorm, partial rotary embedding.

The reference registers two variants selected by ``USE_MCORE_GDN`` (``src/mcore_bridge/model/gpts/qwen3_next.py:594``,
``qwen3_next_gdn.py:153-162``): one wrapping the Hugging Face module (no context parallelism) and one on the
Megatron GDN.  Here there is a single native implementation (``layers/gated_delta_net.py``) that supports
tensor, sequence and context parallelism, so both settings resolve to it.
"""
from ..constant import ModelType
from ..register import ModelMeta, register_model

register_model(ModelMeta(ModelType.qwen3_next, ['qwen3_next']))
