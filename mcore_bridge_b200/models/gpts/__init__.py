from . import llm, qwen3_next  # noqa: F401
