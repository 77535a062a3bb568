"""Text-only families served by the generic ``GPTModel`` + ``GPTBridge`` pair.

Parity: reference ``src/mcore_bridge/model/gpts/llm.py:5-13``.
"""
from ..constant import ModelType
from ..register import ModelMeta, register_model

register_model(
    ModelMeta(ModelType.gpt, [
        'qwen2', 'llama', 'qwen3', 'qwen2_moe', 'qwen3_moe', 'internlm3', 'mimo', 'deepseek', 'deepseek_v2',
        'deepseek_v3', 'deepseek_v32', 'kimi_k2', 'dots1', 'ernie4_5', 'glm4_moe', 'glm4_moe_lite',
        'glm_moe_dsa', 'mistral'
    ]))
