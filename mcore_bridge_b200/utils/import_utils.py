"""Lazy name resolution for the package façade, so ``import mcore_bridge_b200`` stays cheap (same purpose as the lazy
module of reference ``src/mcore_bridge/utils/import_utils.py:11-67``, done with module-level ``__getattr__``)."""
from __future__ import annotations

import importlib
from typing import Any


def lazy_exports(package: str, table: dict[str, list[str]]):
    """PEP 562 hooks (``__getattr__``, ``__dir__``) for a package whose public names live in submodules.

    ``table`` maps a submodule to the names it exports; the submodule is imported the first time one of its names
    (or the submodule itself) is asked for, and the result is cached in the package's namespace.
    """
    owner = {name: sub for sub, names in table.items() for name in names}
    public = sorted(set(table) | set(owner))

    def __getattr__(name: str) -> Any:
        import sys
        if name in table:
            value = importlib.import_module(f'{package}.{name}')
        elif name in owner:
            value = getattr(importlib.import_module(f'{package}.{owner[name]}'), name)
        else:
            raise AttributeError(f'module {package} has no attribute {name}')
        setattr(sys.modules[package], name, value)
        return value

    def __dir__():
        import sys
        return sorted(set(vars(sys.modules[package])) | set(public))

    return __getattr__, __dir__, public


def is_flash_attn_3_available() -> bool:
    return (importlib.util.find_spec('flash_attn_3') is not None
            or importlib.util.find_spec('flash_attn_interface') is not None)
