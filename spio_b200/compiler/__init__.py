"""Just-in-time compilation of the CUDA kernels with NVRTC (sm_100a)."""

from .arch import sm_from_arch
from .compile import compile_cuda, nvrtc_version
from .compile_kernel import compile_kernel, load_kernel, compile_and_load_kernel
from .compiler_pool import compile_kernels, compile_kernel_configs
from .cuda_paths import cuda_include_dir, nvrtc_library_path, kernel_headers
from .flags import lineinfo, debug, workers

__all__ = [
    "sm_from_arch", "compile_cuda", "nvrtc_version", "compile_kernel", "load_kernel",
    "compile_and_load_kernel", "compile_kernels", "compile_kernel_configs", "cuda_include_dir",
    "nvrtc_library_path", "kernel_headers", "lineinfo", "debug", "workers",
]
