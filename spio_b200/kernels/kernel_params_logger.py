"""Records which (kernel, params) pairs a model asks for.

Used by the autotuner to collect the unique layer shapes of a network before it times
tile configurations (reference: spio/kernels/kernel_params_logger.py:22-111).
"""

from __future__ import annotations

import functools
import threading
from typing import Any, Dict, List, Tuple

_lock = threading.Lock()
_active = 0
_records: List[Tuple[Any, Any, Dict[str, Any]]] = []


def kernel_params_logging_is_enabled() -> bool:
    return _active > 0


class KernelParamsLogger:
    """Context manager; inside it every ``KernelCache.get`` call is recorded."""

    def __enter__(self):
        global _active
        with _lock:
            _active += 1
            if _active == 1:
                _records.clear()
        return self

    def __exit__(self, *exc):
        global _active
        with _lock:
            _active -= 1
        return False

    @staticmethod
    def get_logged_params() -> List[Tuple[Any, Any, Dict[str, Any]]]:
        """Unique (kernel_factory, params, kernel_kwargs) triples in first-seen order."""
        seen, out = set(), []
        with _lock:
            for factory, params, kwargs in _records:
                key = (id(factory), params, tuple(sorted(kwargs.items())))
                if key not in seen:
                    seen.add(key)
                    out.append((factory, params, dict(kwargs)))
        return out


def log_kernel_params(method):
    """Decorator for ``KernelCache.get(self, kernel_factory, params, device, **kwargs)``."""

    @functools.wraps(method)
    def wrapper(self, kernel_factory, params, device, **kwargs):
        if _active > 0:
            with _lock:
                _records.append((kernel_factory, params, dict(kwargs)))
        return method(self, kernel_factory, params, device, **kwargs)

    return wrapper
