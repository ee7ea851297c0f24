"""Cache of loaded kernels keyed by (device ordinal, params), with an overlay that lets a
benchmark force specific configurations (reference: spio/kernels/kernel_cache.py:21-111)."""

from __future__ import annotations

from typing import Dict

import torch

from ..cuda.driver import get_device_attributes
from ..util.logger import log
from ..util.tensor_format import get_device_ordinal
from .kernel import Kernel
from .kernel_key import KernelKey
from .kernel_params_logger import kernel_params_logging_is_enabled, log_kernel_params
from .performance_model_cache import PerformanceModelCache

perf_model_cache = PerformanceModelCache()


class KernelCache:
    def __init__(self):
        self._cache: Dict[KernelKey, Kernel] = {}
        self._cache_overlay: Dict[KernelKey, Kernel] = {}

    def update_overlay(self, overlay: Dict[KernelKey, Kernel]) -> None:
        """While an overlay is set only its kernels are used."""
        self._cache_overlay.update(overlay)

    def clear_overlay(self) -> None:
        self._cache_overlay.clear()

    def clear_cache(self) -> None:
        self._cache.clear()

    @log_kernel_params
    def get(self, kernel_factory, params, device, **kernel_kwargs) -> Kernel:
        device = torch.device(device)
        ordinal = get_device_ordinal(device)
        key = KernelKey(device_ordinal=ordinal, params=params)
        if self._cache_overlay:
            kernel = self._cache_overlay.get(key)
            if kernel is None:
                raise ValueError(f"Kernel {kernel_factory} with params {params} and device {device} "
                                 f"not found in overlay cache")
            return kernel
        kernel = self._cache.get(key)
        if kernel is None:
            if kernel_params_logging_is_enabled():
                # shapes are being collected: any valid configuration will do
                config = next(iter(kernel_factory.configs(
                    params, get_device_attributes(ordinal), **kernel_kwargs)))
            else:
                config = perf_model_cache.predict_best_kernel(kernel_factory, params, device,
                                                              **kernel_kwargs)
            kernel = compile_and_load_kernel(kernel_factory, params, config, ordinal, **kernel_kwargs)
            self._cache[key] = kernel
            log(f"loaded kernel {kernel.kernel_name} {config} for device {device}.")
        return kernel


def compile_and_load_kernel(kernel_factory, params, config, device_ordinal: int, **kernel_kwargs) -> Kernel:
    kernel = kernel_factory.make_kernel(params, config, get_device_attributes(device_ordinal),
                                        **kernel_kwargs)
    kernel.compile(get_device_attributes(device_ordinal))
    kernel.load(device_ordinal=device_ordinal)
    return kernel
