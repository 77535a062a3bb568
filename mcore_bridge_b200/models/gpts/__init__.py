from . import llm  # noqa: F401
