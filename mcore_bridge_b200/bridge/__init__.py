from .gpt_bridge import GPTBridge, MultimodalGPTBridge
