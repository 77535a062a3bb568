from . import deepseek_v4, families, llm, qwen3_next  # noqa: F401
