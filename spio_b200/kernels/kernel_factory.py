"""Makes and caches kernels for one CUDA kernel family.

Interface of the reference's ``KernelFactory`` (spio/kernels/kernel_factory.py:79-216):
``configs``, ``get_kernel_name``, ``get_full_kernel_name``, ``get_kernel_cache``,
``get_kernel`` and ``make_kernel``; keyword arguments select the mode of a kernel family
(``igrad=True`` for the input-gradient form of the forward kernel).
"""

from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional, Union

from ..util.tensor_format import check_channels_last
from .kernel import Kernel, get_full_kernel_name


def _wants_jit(params, config) -> bool:
    from ..compiler import flags

    tune = config.as_tune() if config is not None else {}
    if flags.jit.get():
        return True
    if tune.get("engine", 0) == 2:
        return False  # built into the library for every filter size it supports
    wpg, tpw, pps = (tune.get(k, 0) for k in ("wpg", "tpw", "pps"))
    if not (wpg and tpw and pps):
        return False
    from .conv2d_gw8_kernel import compiled_variants

    return (wpg, tpw, pps) not in compiled_variants(params.r, params.s)


class KernelFactory:
    def __init__(self, params_cls=None, config_cls=None, stats_cls=None,
                 kernel_name: Union[str, Callable[..., str]] = None,
                 configs: Union[List[Any], Callable[..., Any]] = None,
                 perf_model_skip_params: Optional[List[str]] = None,
                 args_checker=check_channels_last,
                 fixup: Optional[Callable[..., Any]] = None):
        self.params_cls = params_cls
        self.config_cls = config_cls
        self.stats_cls = stats_cls
        self._kernel_name = kernel_name
        self._configs = configs
        self._args_checker = args_checker
        self._fixup = fixup
        self._kernel_caches: Dict[str, Any] = {}
        self.per_model_skip_params = list(perf_model_skip_params or [])

    def configs(self, params, device_attr, **kwargs):
        """Every valid tile configuration for these layer parameters on this device."""
        if callable(self._configs):
            return self._configs(params, device_attr, **kwargs)
        return self._configs

    def fixup_config(self, params, config, device_attr, **kwargs):
        """A configuration read from a tuning table, adjusted to rules learned after the table
        was measured (identity unless the factory was given a ``fixup``)."""
        if self._fixup is None:
            return config
        return self._fixup(params, config, device_attr, **kwargs)

    def get_kernel_name(self, **kwargs) -> str:
        return self._kernel_name(**kwargs) if callable(self._kernel_name) else self._kernel_name

    def get_full_kernel_name(self, params, **kwargs) -> str:
        return get_full_kernel_name(self.get_kernel_name(**kwargs), params)

    def get_kernel_cache(self, **kwargs):
        from .kernel_cache import KernelCache

        name = self.get_kernel_name(**kwargs)
        cache = self._kernel_caches.get(name)
        if cache is None:
            cache = self._kernel_caches[name] = KernelCache()
        return cache

    def get_kernel(self, params, device, **kwargs) -> Kernel:
        """The best kernel for params on device: cached, else chosen by the performance
        model, made and loaded."""
        return self.get_kernel_cache(**kwargs).get(self, params, device, **kwargs)

    def make_kernel(self, params, config, device_attr=None, jit: Optional[bool] = None, **kwargs) -> Kernel:
        """``jit=True`` compiles the kernel with NVRTC, ``jit=False`` uses a variant built into
        the library; the default is just in time only when SPIO_JIT is set or the
        configuration's (wpg, tpw, pps) is not among the built-in variants."""
        del device_attr
        if jit is None:
            jit = _wants_jit(params, config)
        cls = Kernel
        if jit:
            from .jit_kernel import JitKernel as cls
        return cls(self.get_full_kernel_name(params, **kwargs), self.get_kernel_name(**kwargs),
                   params=params, config=config, args_checker=self._args_checker)

    def __repr__(self) -> str:
        return f"KernelFactory({self._kernel_name if isinstance(self._kernel_name, str) else 'conv2d_gw8'})"
