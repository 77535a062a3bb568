"""Small generic helpers (parity: reference ``src/mcore_bridge/utils/utils.py:15-106``)."""
from __future__ import annotations

import json
import os
from contextlib import contextmanager
from typing import Callable, Dict, Optional, TypeVar, Union

_T = TypeVar('_T')


def json_parse_to_dict(value: Union[str, Dict, None], strict: bool = True) -> Union[str, Dict, None]:
    """Accepts a dict, a JSON string or a path to a JSON file; returns a dict."""
    if value is None:
        return {}
    if isinstance(value, dict):
        return value
    if isinstance(value, str):
        if os.path.exists(value):
            with open(value, 'r', encoding='utf-8') as f:
                return json.load(f)
        try:
            return json.loads(value)
        except json.JSONDecodeError:
            if strict:
                raise ValueError(f'cannot parse {value!r} as JSON')
            return value
    raise TypeError(f'unsupported type {type(value)}')


def get_env_args(args_name: str, type_func: Callable[[str], _T], default_value: Optional[_T]) -> Optional[_T]:
    """Reads ``ARGS_NAME`` (upper- or lower-case) from the environment and converts it."""
    raw = os.getenv(args_name.upper())
    if raw is None:
        raw = os.getenv(args_name.lower())
    if raw is None:
        return default_value
    if type_func is bool:
        return raw.strip().lower() in {'1', 'true', 'yes', 'on'}
    return type_func(raw)


def deep_getattr(obj, attr: str, default=None):
    for name in attr.split('.'):
        if obj is None:
            return default
        if isinstance(obj, dict):
            obj = obj.get(name, default)
        else:
            obj = getattr(obj, name, default)
    return obj


@contextmanager
def patch_deepcopy():
    """Deep-copies modules while sharing process groups and config objects (they are not copyable).

    Used when an adapter wrapper clones a module tree (``modules_to_save``): the clone must keep the
    same ``ProcessGroup`` handles and the same ``ModelConfig`` instance.
    """
    import torch.distributed as dist
    originals = {}
    pg_cls = getattr(dist, 'ProcessGroup', None)
    from ..config.model_config import ModelConfig
    for cls in filter(None, [pg_cls]):
        originals[cls] = cls.__dict__.get('__deepcopy__')
        cls.__deepcopy__ = lambda self, memo: self
    saved_cfg = ModelConfig.__dict__.get('__deepcopy__')
    ModelConfig.__deepcopy__ = lambda self, memo: self
    try:
        yield
    finally:
        for cls, fn in originals.items():
            if fn is None:
                try:
                    delattr(cls, '__deepcopy__')
                except (AttributeError, TypeError):
                    pass
            else:
                cls.__deepcopy__ = fn
        if saved_cfg is None:
            del ModelConfig.__deepcopy__
        else:
            ModelConfig.__deepcopy__ = saved_cfg
