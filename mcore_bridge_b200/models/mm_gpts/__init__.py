from . import qwen, vision_families  # noqa: F401
