from . import families, llm, qwen3_next  # noqa: F401
