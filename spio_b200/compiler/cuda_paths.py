"""Where NVRTC, the CUDA headers and the kernel headers of this package are.

The reference takes the CUDA runtime headers from the ``nvidia.cuda_runtime`` wheel and
NVRTC from the ``nvidia.cuda_nvrtc`` wheel (spio/compiler/compile.py:14-18,
spio/cuda/nvrtc_ctypes.py:19-40).  Both are looked for here as well, after the environment
variables SPIO_NVRTC / SPIO_CUDA_INCLUDE and before a CUDA toolkit under CUDA_HOME or
/usr/local/cuda.
"""

from __future__ import annotations

import importlib.util
import os
from functools import lru_cache
from pathlib import Path
from typing import Dict, List, Optional

CSRC_DIR = Path(__file__).resolve().parent.parent / "csrc"

# The device-only headers a kernel translation unit includes.
KERNEL_HEADER_NAMES = ("ptx.cuh", "gw8_common.cuh", "conv2d_gw8_fwd.cuh", "conv2d_gw8_wgrad.cuh",
                       "conv2d_gw8_fwd_tc.cuh", "typed.h", "typed_tma.cuh", "typed_mma.cuh")


def _package_dir(name: str) -> Optional[Path]:
    try:
        spec = importlib.util.find_spec(name)
    except (ImportError, ValueError):
        return None
    if spec is None or not spec.submodule_search_locations:
        return None
    return Path(list(spec.submodule_search_locations)[0])


def _toolkit_roots() -> List[Path]:
    roots = [os.environ.get(k) for k in ("CUDA_HOME", "CUDA_PATH")]
    return [Path(r) for r in roots if r] + [Path("/usr/local/cuda")]


@lru_cache(maxsize=None)
def nvrtc_library_path() -> str:
    """Full path of libnvrtc.so.12; raises FileNotFoundError if there is none."""
    env = os.environ.get("SPIO_NVRTC")
    candidates = [Path(env)] if env else []
    candidates += [root / "lib64" / "libnvrtc.so.12" for root in _toolkit_roots()]
    wheel = _package_dir("nvidia.cuda_nvrtc")
    if wheel is not None:
        candidates.append(wheel / "lib" / "libnvrtc.so.12")
    for cand in candidates:
        if cand.exists():
            return str(cand)
    raise FileNotFoundError("libnvrtc.so.12 not found; set SPIO_NVRTC to its path")


@lru_cache(maxsize=None)
def cuda_include_dir() -> str:
    """Directory that holds cuda_fp16.h."""
    env = os.environ.get("SPIO_CUDA_INCLUDE")
    candidates = [Path(env)] if env else []
    candidates += [root / "include" for root in _toolkit_roots()]
    wheel = _package_dir("nvidia.cuda_runtime")
    if wheel is not None:
        candidates.append(wheel / "include")
    for cand in candidates:
        if (cand / "cuda_fp16.h").exists():
            return str(cand)
    raise FileNotFoundError("cuda_fp16.h not found; set SPIO_CUDA_INCLUDE to the CUDA include directory")


@lru_cache(maxsize=None)
def _kernel_headers() -> Dict[str, str]:
    return {name: (CSRC_DIR / name).read_text() for name in KERNEL_HEADER_NAMES}


def kernel_headers() -> Dict[str, str]:
    """name -> text of the kernel headers, handed to NVRTC in memory."""
    return dict(_kernel_headers())
