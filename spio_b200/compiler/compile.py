"""Compile CUDA source text to a cubin with NVRTC.

Same job and arguments as the reference's ``compile_cuda`` (spio/compiler/compile.py:22-77),
which drives NVRTC through a ctypes ``Program`` class (spio/cuda/nvrtc_ctypes.py:152-217).
Here the NVRTC calls are made by the native library (``spio_jit_compile``); ctypes releases
the interpreter lock for the duration of the call, so several compilations run in parallel
on threads of one process.
"""

from __future__ import annotations

import ctypes
from pathlib import Path
from typing import Dict, List, Optional, Tuple, Union

from .. import _clib
from .arch import sm_from_arch
from .cuda_paths import cuda_include_dir, nvrtc_library_path

_nvrtc_ready = False


def _lib():
    global _nvrtc_ready
    lib = _clib.load()
    if not _nvrtc_ready:
        _clib.check(lib.spio_jit_set_nvrtc_path(nvrtc_library_path().encode()), "nvrtc")
        _nvrtc_ready = True
    return lib


def nvrtc_version() -> Tuple[int, int]:
    major, minor = ctypes.c_int(), ctypes.c_int()
    _clib.check(_lib().spio_jit_nvrtc_version(ctypes.byref(major), ctypes.byref(minor)), "nvrtc")
    return major.value, minor.value


def _c_strings(items: List[str]):
    arr = (ctypes.c_char_p * max(len(items), 1))()
    for i, text in enumerate(items):
        arr[i] = text.encode()
    return arr


def compile_cuda(
    src: Union[str, Path],
    includes: Optional[List[str]] = None,
    arch: Union[Tuple[int, int], str, None] = None,
    device_debug: bool = False,
    lineinfo: bool = False,
    header_dict: Optional[Dict[str, str]] = None,
    max_registers: Optional[int] = None,
    default_device: bool = False,
    src_name: Optional[str] = None,
    ptxas_verbose: bool = False,
    return_log: bool = False,
    defines: Optional[Dict[str, object]] = None,
):
    """Compile ``src`` (a path, or the source text itself together with ``src_name``) and
    return the cubin as bytes, or ``(cubin, log)`` with ``return_log``.

    Raises ``ValueError("Compilation error log: ...")`` when NVRTC rejects the program.
    """
    if isinstance(src, Path):
        text, name = src.read_text(), src_name or src.name
    else:
        text, name = src, src_name or "kernel.cu"
    options = ["-std=c++17"]
    sm = sm_from_arch(arch)
    if sm is not None:
        options.append(f"-arch={sm}")
    if device_debug:
        options.append("-G")
    if lineinfo:
        options.append("-lineinfo")
    if max_registers is not None:
        options.append(f"-maxrregcount={max_registers}")
    if default_device:
        options.append("-default-device")
    if ptxas_verbose:
        options.append("--ptxas-options=-v")
    for macro, value in (defines or {}).items():
        options.append(f"-D{macro}" if value is None else f"-D{macro}={value}")
    options += [f"-I{path}" for path in (includes or []) + [cuda_include_dir()]]

    header_dict = header_dict or {}
    names, sources = list(header_dict.keys()), list(header_dict.values())
    cubin, size, log = ctypes.c_void_p(), ctypes.c_size_t(), ctypes.c_void_p()
    lib = _lib()
    rc = lib.spio_jit_compile(text.encode(), name.encode(), _c_strings(options), len(options),
                              _c_strings(names), _c_strings(sources), len(names),
                              ctypes.byref(cubin), ctypes.byref(size), ctypes.byref(log))
    log_text = ""
    if log.value:
        log_text = ctypes.string_at(log.value).decode(errors="replace")
        lib.spio_jit_free(log)
    if rc != 0:
        cause = lib.spio_b200_last_error().decode(errors="replace")
        raise ValueError(f"Compilation error log: {log_text or cause}")
    image = ctypes.string_at(cubin.value, size.value)
    lib.spio_jit_free(cubin)
    return (image, log_text) if return_log else image
