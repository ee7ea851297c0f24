"""The binding a maintainer of the reference would add to use libspio_b200 (the integration guide shows it).

Drop this file into the reference as ``spio/kernels/b200_kernel.py``: :class:`B200Kernel` has the call
protocol of the reference's ``spio.kernels.Kernel`` (``compile`` / ``load`` / ``__call__`` with the
tensors in the order the reference's kernels take them, spio/kernels/kernel.py:37-157) and forwards
to the C ABI of the library through ctypes.  It imports nothing from this package, only the shared
library; ``tests/test_reference_binding_gpu.py`` runs it against the CPU oracle.
"""

import ctypes
import os

import torch

_LIB_PATH = os.environ.get("SPIO_B200_LIB") or os.path.join(
    os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib", "libspio_b200.so")
_lib = ctypes.CDLL(_LIB_PATH)            # libspio_b200.so
_lib.spio_conv2d_gw8_wgrad_scratch_bytes.restype = ctypes.c_size_t
_lib.spio_b200_last_error.restype = ctypes.c_char_p


class _Shape(ctypes.Structure):
    _fields_ = [(k, ctypes.c_int) for k in ("n", "c", "h", "w", "r", "s", "pad_h", "pad_w")]


def _shape(p):  # p: spio.kernels.Conv2dGw8Params
    return _Shape(p.n, p.c, p.h, p.w, p.r, p.s, p.padding_h, p.padding_w)


class B200Kernel:
    """Same call protocol as spio.kernels.Kernel; ``kernel_name`` is the reference's full kernel name
    (``spio_conv2d_gw8_fprop__...``, ``..._dgrad__...`` or ``..._wgrad__...``)."""

    def __init__(self, kernel_name, params):
        self.kernel_name, self.params, self._sh = kernel_name, params, _shape(params)
        self._scratch = None

    def compile(self):
        pass  # the kernels are compiled ahead of time into the library

    def load(self, device_ordinal=0, clear_cubin=True):
        pass

    def __call__(self, *args):
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        ptr = [ctypes.c_void_p(a.data_ptr()) if a is not None else None for a in args]
        sh = ctypes.byref(self._sh)
        if "fprop" in self.kernel_name:      # (output, input, weight, bias)
            rc = _lib.spio_conv2d_gw8_fprop(ptr[0], ptr[1], ptr[2], ptr[3], sh, None, stream)
        elif "dgrad" in self.kernel_name:    # (grad_input, grad_output, weight, None)
            rc = _lib.spio_conv2d_gw8_dgrad(ptr[0], ptr[1], ptr[2], sh, None, stream)
        else:                                # (grad_weight, input, grad_output); grad_weight need not be zeroed
            n = _lib.spio_conv2d_gw8_wgrad_scratch_bytes(sh, None)
            if self._scratch is None or self._scratch.numel() < n:
                self._scratch = torch.empty(n, dtype=torch.uint8, device=args[0].device)
            rc = _lib.spio_conv2d_gw8_wgrad(ptr[0], ptr[1], ptr[2], sh, None,
                                            ctypes.c_void_p(self._scratch.data_ptr()), ctypes.c_size_t(n), stream)
        if rc:
            raise ValueError(_lib.spio_b200_last_error().decode())
