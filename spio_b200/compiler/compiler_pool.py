"""Compile many kernels in parallel.

The reference forks a pool of SPIO_WORKERS processes at import time
(spio/compiler/compiler_pool.py:25-86).  NVRTC is thread-safe and the native compile call
runs without the interpreter lock, so a thread pool made on first use does the same job
without forking a process that may already hold a CUDA context.
"""

from __future__ import annotations

from concurrent.futures import ThreadPoolExecutor
from typing import Any, List, Optional, Tuple

from . import flags

_pool: Optional[ThreadPoolExecutor] = None


def _get_pool() -> ThreadPoolExecutor:
    global _pool
    if _pool is None:
        _pool = ThreadPoolExecutor(max_workers=flags.workers, thread_name_prefix="spio-nvrtc")
    return _pool


def compile_kernels(kernels: List[Any], arch: Tuple[int, int] = None) -> None:
    """Compile every kernel (objects with a ``compile`` method); afterwards each has its cubin."""
    del arch  # each kernel knows the architecture it was made for
    if not kernels:
        return
    try:
        list(_get_pool().map(lambda k: k.compile(), kernels))
    except Exception as exc:
        raise ValueError("Error compiling kernels") from exc


def compile_kernel_configs(kernel_factory, params, configs: Optional[List[Any]] = None, device_attr=None,
                           **kernel_kwargs) -> List[Any]:
    """Make and compile one kernel per configuration (all valid ones if none are given).
    ``load`` each returned kernel on a device before launching it."""
    from ..cuda.driver import B200_ATTRIBUTES

    device_attr = device_attr or B200_ATTRIBUTES
    if configs is None:
        configs = list(kernel_factory.configs(params, device_attr, **kernel_kwargs))
    kernels = [kernel_factory.make_kernel(params, config=c, device_attr=device_attr, **kernel_kwargs)
               for c in configs]
    compile_kernels(kernels, arch=device_attr.compute_capability)
    return kernels
