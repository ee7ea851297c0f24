"""A kernel bound to one problem shape and one tile configuration.

Mirrors the reference's ``Kernel`` (spio/kernels/kernel.py:37-157): objects are made by
a :class:`KernelFactory`, go through ``compile()`` and ``load()`` and are then called with
tensors.  Here the device code lives ahead-of-time compiled in libspio_b200.so and a call
goes through its C ABI on torch's current stream; ``compile()`` checks that the shape and
configuration can be planned, ``load()`` loads the library.  There is no fallback: a
missing library or device raises.
"""

from __future__ import annotations

import ctypes
from typing import Any, Optional

import torch

from .. import _clib
from ..util.tensor_format import check_channels_last
from .launch_params import LaunchParams

KIND_BY_NAME = {
    "spio_conv2d_gw8_fprop": _clib.FPROP,
    "spio_conv2d_gw8_dgrad": _clib.DGRAD,
    "spio_conv2d_gw8_wgrad": _clib.WGRAD,
}


def get_full_kernel_name(kernel_name: str, params) -> str:
    """``<kernel>__<encoded params>`` (reference: spio/kernels/kernel.py:160-163)."""
    return f"{kernel_name}__{params.encode()}"


def shape_of(params) -> _clib.Shape:
    return _clib.Shape(params.n, params.c, params.h, params.w, params.r, params.s,
                       params.padding_h, params.padding_w)


# Weight-gradient scratch, one buffer per (device, stream): kernels of one stream run in order (the
# weight-gradient kernel never skips its dependency wait), so they can share it; kernels of
# different streams cannot.  Buffers only grow; outgrown ones are kept alive because a recorded
# CUDA graph may still hold their address.
_scratch: dict = {}
_outgrown: list = []


def scratch_for(device, stream_ptr: int, nbytes: int) -> torch.Tensor:
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream_ptr)
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        if buf is not None:
            _outgrown.append(buf)
        buf = _scratch[key] = torch.empty(max(nbytes, 4 << 20), dtype=torch.uint8, device=device)
    return buf


class Kernel:
    def __init__(self, kernel_name: str, base_name: str, params, config=None,
                 args_checker=check_channels_last):
        self.kernel_name = kernel_name
        self.base_name = base_name
        self.kind = KIND_BY_NAME[base_name]
        self.params = params
        self.config = config
        self._args_checker = args_checker
        self._shape = shape_of(params)
        self._tune = _clib.make_tune(config.as_tune() if config is not None else None)
        self._lib = None
        self._device_ordinal: Optional[int] = None
        self._scratch_bytes = 0
        self.plan = None

    # ------------------------------------------------------------ life cycle
    def _tune_ref(self):
        return ctypes.byref(self._tune) if self._tune is not None else None

    def compile(self, device_attr=None) -> None:
        """Validate shape + configuration by planning the launch (no device needed when
        device attributes are given)."""
        from ..cuda.driver import B200_ATTRIBUTES

        attr = device_attr or B200_ATTRIBUTES
        lib = _clib.load()
        info = _clib.PlanInfo()
        _clib.check(lib.spio_conv2d_gw8_plan_for(
            self.kind, ctypes.byref(self._shape), self._tune_ref(), attr.multiprocessor_count,
            attr.max_shared_memory_per_block_optin, ctypes.byref(info)), self.kernel_name)
        self.plan = info.as_dict()

    def load(self, device_ordinal: int = 0, clear_cubin: bool = True) -> None:
        del clear_cubin  # the device code is part of the shared library
        if not torch.cuda.is_available():
            raise ValueError("CUDA error: no CUDA device is available")
        self._lib = _clib.load()
        self._device_ordinal = device_ordinal
        with torch.cuda.device(device_ordinal):
            info = _clib.PlanInfo()
            _clib.check(self._lib.spio_conv2d_gw8_plan(
                self.kind, ctypes.byref(self._shape), self._tune_ref(), ctypes.byref(info)),
                self.kernel_name)
        self.plan = info.as_dict()
        self._scratch_bytes = int(info.scratch_bytes)

    def unload(self) -> None:
        self._lib = None
        self._device_ordinal = None

    @property
    def launch_params(self) -> Optional[LaunchParams]:
        if self.plan is None:
            return None
        return LaunchParams(self.plan["grid"], self.plan["threads"], self.plan["smem_bytes"])

    # ------------------------------------------------------------ launch
    def launch(self, *args) -> None:
        """fprop: (output, input, weight, bias|None); dgrad: (grad_input, grad_output, weight,
        None); wgrad: (grad_weight, input, grad_output).  Tensors are channels_last."""
        if self._lib is None:
            raise ValueError(f"Error in kernel {self}: kernel is not loaded")
        try:
            self._args_checker(args)
            dev = args[0].device
            stream = torch.cuda.current_stream(dev).cuda_stream
            ptr = [a.data_ptr() if a is not None else None for a in args]
            sh, tn = ctypes.byref(self._shape), self._tune_ref()
            with torch.cuda.device(dev):
                if self.kind == _clib.FPROP:
                    rc = self._lib.spio_conv2d_gw8_fprop(ptr[0], ptr[1], ptr[2], ptr[3], sh, tn, stream)
                elif self.kind == _clib.DGRAD:
                    rc = self._lib.spio_conv2d_gw8_dgrad(ptr[0], ptr[1], ptr[2], sh, tn, stream)
                else:
                    scratch = scratch_for(dev, stream, self._scratch_bytes)
                    rc = self._lib.spio_conv2d_gw8_wgrad(ptr[0], ptr[1], ptr[2], sh, tn,
                                                         scratch.data_ptr(), self._scratch_bytes, stream)
            _clib.check(rc)
        except Exception as exc:
            raise ValueError(f"Error in kernel {self}: {exc}") from exc

    __call__ = launch

    def __repr__(self) -> str:
        return f"{self.kernel_name} {self.config}"


def launch_backward(wgrad_kernel: Kernel, dgrad_kernel: Optional[Kernel], grad_input, grad_weight, inputs,
                    grad_output, weight, grad_bias=None) -> None:
    """Weight gradient, optionally the bias gradient (odd number of filter taps only) and,
    with ``dgrad_kernel``, the input gradient of a layer, through the library's combined entry
    point: weight gradient, reduce and input gradient are chained with programmatic dependent
    launch.  Kernels built into the library and kernels compiled just in time mix freely; the
    latter are passed by their function handles.  ``grad_weight`` may be fp32 (the reference's
    contract) or fp16 (the parameter's own type, rounded once from the fp32 sum)."""
    kernels = [wgrad_kernel] + ([dgrad_kernel] if dgrad_kernel is not None else [])
    for k in kernels:
        if k._lib is None:
            raise ValueError(f"Error in kernel {k}: kernel is not loaded")
    try:
        wgrad_kernel._args_checker((grad_weight, inputs, grad_output))
        if dgrad_kernel is not None:
            dgrad_kernel._args_checker((grad_input, grad_output, weight, None))
        if grad_weight.dtype not in (torch.float32, torch.float16):
            raise ValueError("grad_weight must be float32 or float16")
        dev = inputs.device
        stream = torch.cuda.current_stream(dev).cuda_stream
        nbytes = wgrad_kernel._scratch_bytes
        opts = _clib.BackwardOpts(
            1 if grad_weight.dtype == torch.float16 else 0,
            getattr(wgrad_kernel, "function_handle", None),
            getattr(wgrad_kernel, "dbias_function_handle", None),
            getattr(dgrad_kernel, "function_handle", None) if dgrad_kernel is not None else None)
        with torch.cuda.device(dev):
            scratch = scratch_for(dev, stream, nbytes)
            rc = wgrad_kernel._lib.spio_conv2d_gw8_backward_ex(
                grad_input.data_ptr() if dgrad_kernel is not None else None, grad_weight.data_ptr(),
                grad_bias.data_ptr() if grad_bias is not None else None, inputs.data_ptr(),
                grad_output.data_ptr(), weight.data_ptr(), ctypes.byref(wgrad_kernel._shape),
                dgrad_kernel._tune_ref() if dgrad_kernel is not None else None,
                wgrad_kernel._tune_ref(), scratch.data_ptr(), nbytes, stream, None, ctypes.byref(opts))
        _clib.check(rc)
    except Exception as exc:
        raise ValueError(f"Error in kernels {wgrad_kernel}, {dgrad_kernel}: {exc}") from exc


def device_status() -> int:
    """Synchronise and return the kernels' status word of the current device (0 = ok)."""
    return _clib.device_status()
