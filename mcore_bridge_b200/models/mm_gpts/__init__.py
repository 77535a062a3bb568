from . import gemma4, qwen, vision_families  # noqa: F401
