"""Kernel layer: shape parameters, statistics, tile configurations, factories and caches
(the names the reference exports from spio.kernels)."""

from .conv2d_gw8_params import Conv2dGw8Params
from .conv2d_stats import Conv2dStats
from .stats import Stats
from .launch_params import LaunchParams
from .kernel import Kernel, get_full_kernel_name, device_status
from .kernel_key import KernelKey
from .kernel_factory import KernelFactory
from .kernel_cache import KernelCache
from .kernel_params_logger import KernelParamsLogger
from .performance_model_cache import PerformanceModelCache
from .conv2d_gw8_kernel import Conv2dGw8Config, conv2d_gw8_kernel_factory
from .conv2d_gw8_wgrad_kernel import Conv2dGw8WgradConfig, conv2d_gw8_wgrad_kernel_factory
