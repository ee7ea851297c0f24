"""ctypes binding of libspio_b200.so, the C-ABI library declared in include/spio_b200.h.

Takes the place of the reference's Cython driver module (spio/cuda/driver.pyx) as the
one native boundary of the package.  There is no CPU fallback: if the library is missing
or fails to load, every operator raises.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_longlong, c_size_t, c_ulonglong, c_void_p
from pathlib import Path
from typing import Optional

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libspio_b200.so"

FPROP, DGRAD, WGRAD = 0, 1, 2


class Shape(Structure):
    """struct spio_gw8_shape."""

    _fields_ = [(k, c_int) for k in ("n", "c", "h", "w", "r", "s", "pad_h", "pad_w")]


class Tune(Structure):
    """struct spio_gw8_tune; zero fields are chosen by the library."""

    _fields_ = [(k, c_int) for k in ("wpg", "tpw", "ns", "nob", "ncb", "nb", "grid", "pps", "engine")]


class PlanInfo(Structure):
    """struct spio_gw8_plan_info."""

    _fields_ = [
        (k, c_int)
        for k in (
            "wpg", "tpw", "ns", "nob", "ncb", "nb", "grid", "threads", "pps", "smem_bytes",
            "n_chunks", "n_image_groups", "n_col_tiles", "n_pairs", "n_split", "engine",
        )
    ] + [("scratch_bytes", c_size_t)]

    def as_dict(self):
        return {name: getattr(self, name) for name, _ in self._fields_}


class DpExchange(Structure):
    """struct spio_dp_exchange."""

    _fields_ = [("buffers", POINTER(c_void_p)), ("rank", c_int), ("world", c_int), ("seq", ctypes.c_uint),
                ("capacity", c_size_t)]


class BackwardOpts(Structure):
    """struct spio_gw8_backward_opts."""

    _fields_ = [("dw_f16", c_int), ("wgrad_function", c_void_p), ("wgrad_dbias_function", c_void_p),
                ("dgrad_function", c_void_p), ("dp", POINTER(DpExchange))]


class Launch(Structure):
    """struct spio_gw8_launch: tensor maps, geometry and launch dimensions of one call of a
    just-in-time compiled kernel."""

    _fields_ = [
        ("in_map", c_ulonglong * 16),
        ("out_map", c_ulonglong * 16),
        ("row_map", c_ulonglong * 16),
        ("geom", c_int * 40),
        ("ns", c_int), ("nob", c_int), ("grid", c_int), ("threads", c_int),
        ("smem_bytes", c_int), ("n_parts", c_int),
        ("scratch_bytes", c_size_t),
        ("status", c_void_p),
    ]


# name -> (restype, argtypes); one entry per symbol declared in include/spio_b200.h
SIGNATURES = {
    "spio_conv2d_gw8_fprop": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune), c_void_p]),
    "spio_conv2d_gw8_dgrad": (
        c_int, [c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune), c_void_p]),
    "spio_conv2d_gw8_wgrad_scratch_bytes": (c_size_t, [POINTER(Shape), POINTER(Tune)]),
    "spio_conv2d_gw8_wgrad": (
        c_int,
        [c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune), c_void_p, c_size_t, c_void_p]),
    "spio_conv2d_gw8_backward": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune), POINTER(Tune),
         c_void_p, c_size_t, c_void_p, c_void_p]),
    "spio_conv2d_gw8_backward_ex": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune), POINTER(Tune),
         c_void_p, c_size_t, c_void_p, c_void_p, POINTER(BackwardOpts)]),
    "spio_conv2d_gw8_fprop_jit": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune), c_void_p]),
    "spio_conv2d_gw8_dgrad_jit": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune), c_void_p]),
    "spio_conv2d_gw8_wgrad_jit": (
        c_int,
        [c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune), c_void_p, c_size_t, c_void_p]),
    "spio_conv2d_gw8_wgrad_scratch_bytes_jit": (c_size_t, [POINTER(Shape), POINTER(Tune)]),
    "spio_dp_buffer_bytes": (c_size_t, [c_int, c_size_t]),
    "spio_dp_buffer_alloc": (c_int, [c_size_t, POINTER(c_void_p), c_void_p]),
    "spio_dp_buffer_open": (c_int, [c_void_p, POINTER(c_void_p)]),
    "spio_dp_buffer_close": (c_int, [c_void_p]),
    "spio_dp_buffer_free": (c_int, [c_void_p]),
    "spio_dp_push": (c_int, [POINTER(DpExchange), c_void_p, c_size_t, c_void_p, c_size_t, c_void_p]),
    "spio_dp_sum": (c_int, [POINTER(DpExchange), c_void_p, c_size_t, c_void_p, c_size_t, c_void_p]),
    "spio_dp_allreduce": (c_int, [POINTER(DpExchange), c_void_p, c_size_t, c_void_p, c_size_t, c_void_p]),
    "spio_conv2d_gw8_wgrad_static": (
        c_int, [c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune), c_void_p]),
    "spio_conv2d_gw8_fprop_host": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune)]),
    "spio_conv2d_gw8_dgrad_host": (
        c_int, [c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune)]),
    "spio_conv2d_gw8_wgrad_host": (
        c_int, [c_void_p, c_void_p, c_void_p, POINTER(Shape), POINTER(Tune)]),
    "spio_conv2d_gw8_step_host": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Shape)]),
    "spio_conv2d_gw8_step_host_dp": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, POINTER(Shape),
                POINTER(DpExchange)]),
    "spio_conv2d_gw8_plan": (c_int, [c_int, POINTER(Shape), POINTER(Tune), POINTER(PlanInfo)]),
    "spio_conv2d_gw8_plan_for": (
        c_int, [c_int, POINTER(Shape), POINTER(Tune), c_int, c_int, POINTER(PlanInfo)]),
    "spio_jit_set_nvrtc_path": (c_int, [c_char_p]),
    "spio_jit_nvrtc_version": (c_int, [POINTER(c_int), POINTER(c_int)]),
    "spio_jit_compile": (
        c_int,
        [c_char_p, c_char_p, POINTER(c_char_p), c_int, POINTER(c_char_p), POINTER(c_char_p), c_int,
         POINTER(c_void_p), POINTER(c_size_t), POINTER(c_void_p)]),
    "spio_jit_free": (None, [c_void_p]),
    "spio_module_load": (c_int, [c_void_p, POINTER(c_void_p)]),
    "spio_module_unload": (c_int, [c_void_p]),
    "spio_module_get_function": (c_int, [c_void_p, c_char_p, POINTER(c_void_p)]),
    "spio_function_set_max_dynamic_smem": (c_int, [c_void_p, c_int]),
    "spio_function_get_attribute": (c_int, [c_void_p, c_int, POINTER(c_int)]),
    "spio_function_launch": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, POINTER(c_void_p)]),
    "spio_function_launch_ex": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, POINTER(c_void_p), c_int]),
    "spio_conv2d_gw8_plan_jit": (
        c_int, [c_int, POINTER(Shape), POINTER(Tune), c_int, c_int, POINTER(PlanInfo)]),
    "spio_conv2d_gw8_prepare_launch": (
        c_int, [c_int, POINTER(Shape), POINTER(Tune), c_void_p, c_void_p, POINTER(Launch)]),
    "spio_conv2d_gw8_wgrad_reduce": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p]),
    "spio_layernorm_2d_fwd": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_float, c_void_p]),
    "spio_layernorm_2d_bwd_scratch_bytes": (c_size_t, [c_longlong, c_int]),
    "spio_layernorm_2d_bwd": (
        c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_longlong, c_int,
                c_void_p, c_size_t, c_void_p]),
    "spio_conv2d_gw8_num_variants": (c_int, []),
    "spio_conv2d_gw8_variant": (
        c_int, [c_int, POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int), POINTER(c_int)]),
    "spio_b200_device_status": (c_int, [POINTER(c_int)]),
    "spio_b200_status_address": (c_int, [POINTER(c_void_p)]),
    "spio_tensor_map_encode": (
        c_int, [c_void_p, c_void_p, c_int, c_int, POINTER(c_ulonglong), POINTER(c_ulonglong),
                POINTER(ctypes.c_uint), c_int]),
    "spio_b200_last_error": (c_char_p, []),
    "spio_b200_version": (c_char_p, []),
}

_lib: Optional[ctypes.CDLL] = None


def load() -> ctypes.CDLL:
    """Load the library once and attach the argument types."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m spio_b200.build` "
            "(there is no fallback implementation)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def last_error() -> str:
    return load().spio_b200_last_error().decode()


def check(rc: int, what: str = "") -> None:
    """Raise ValueError (the reference's convention for CUDA errors,
    spio/cuda/driver.pyx:118-123) when a call returned non-zero."""
    if rc != 0:
        msg = last_error()
        raise ValueError(f"{msg}" + (f" [{what}]" if what else ""))


def make_tune(tune) -> Optional[Tune]:
    """Accept None, a Tune, or a mapping / object with the tune's field names."""
    if tune is None:
        return None
    if isinstance(tune, Tune):
        return tune
    if isinstance(tune, dict):
        return Tune(**{k: int(v) for k, v in tune.items()})
    return Tune(**{k: int(getattr(tune, k, 0)) for k, _ in Tune._fields_})


def tune_ref(tune):
    t = make_tune(tune)
    return ctypes.byref(t) if t is not None else None


def device_status() -> int:
    """Synchronise the current device and return (and clear) its kernel status word."""
    st = c_int(0)
    check(load().spio_b200_device_status(ctypes.byref(st)), "device_status")
    return st.value
