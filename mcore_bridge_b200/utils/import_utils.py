"""Lazy module used by the package façade so ``import mcore_bridge_b200`` stays cheap.

Parity: reference ``src/mcore_bridge/utils/import_utils.py:11-67``.
"""
from __future__ import annotations

import importlib
import os
from itertools import chain
from types import ModuleType
from typing import Any


class _LazyModule(ModuleType):
    """Resolves ``package.Name`` on first access from an ``{submodule: [names]}`` table."""

    def __init__(self, name, module_file, import_structure, module_spec=None, extra_objects=None):
        super().__init__(name)
        self._modules = set(import_structure.keys())
        self._class_to_module = {}
        for key, values in import_structure.items():
            for value in values:
                self._class_to_module[value] = key
        self.__all__ = list(import_structure.keys()) + list(chain(*import_structure.values()))
        self.__file__ = module_file
        self.__spec__ = module_spec
        self.__path__ = [os.path.dirname(module_file)]
        self._objects = {} if extra_objects is None else extra_objects
        self._name = name
        self._import_structure = import_structure

    def __dir__(self):
        result = list(super().__dir__())
        result.extend(a for a in self.__all__ if a not in result)
        return result

    def __getattr__(self, name: str) -> Any:
        if name in self._objects:
            return self._objects[name]
        if name in self._modules:
            value = self._get_module(name)
        elif name in self._class_to_module:
            value = getattr(self._get_module(self._class_to_module[name]), name)
        else:
            raise AttributeError(f'module {self.__name__} has no attribute {name}')
        setattr(self, name, value)
        return value

    def _get_module(self, module_name: str):
        return importlib.import_module('.' + module_name, self.__name__)

    def __reduce__(self):
        return self.__class__, (self._name, self.__file__, self._import_structure)


def is_flash_attn_3_available() -> bool:
    return importlib.util.find_spec('flash_attn_3') is not None or importlib.util.find_spec('flash_attn_interface') is not None
