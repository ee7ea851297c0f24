"""A kernel compiled just in time with NVRTC and launched through the driver API.

Mirrors the reference's kernel life cycle (spio/kernels/kernel.py:37-157): ``compile()``
turns generated source into a cubin, ``load()`` loads the cubin into the device's primary
context and looks the function up by its full name, ``launch()`` passes the tensors.  The
instantiated tile configuration does not have to be one of those built into the library,
which is what the autotuner uses to search beyond them.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .. import _clib
from ..util.tensor_format import check_channels_last
from .kernel import KIND_BY_NAME, Kernel
from .launch_params import LaunchParams


class JitKernel(Kernel):
    def __init__(self, kernel_name: str, base_name: str, params, config=None,
                 args_checker=check_channels_last):
        super().__init__(kernel_name, base_name, params, config, args_checker)
        self.cubin: Optional[bytes] = None
        self.compile_log: str = ""
        self.module = None
        self.function = None
        self.dbias_function = None  # weight gradient only: the instantiation that also sums dy
        self._arch = None

    # ------------------------------------------------------------ life cycle
    def _resolve_tune(self, attr) -> None:
        """Fill wpg / tpw / pps from the launch planner when the configuration leaves them open."""
        t = self._tune
        if t is not None and (t.engine == 2 or (t.wpg > 0 and t.tpw > 0 and t.pps > 0)):
            return
        info = _clib.PlanInfo()
        _clib.check(_clib.load().spio_conv2d_gw8_plan_for(
            self.kind, ctypes.byref(self._shape), self._tune_ref(), attr.multiprocessor_count,
            attr.max_shared_memory_per_block_optin, ctypes.byref(info)), self.kernel_name)
        if t is None:
            t = self._tune = _clib.Tune()
        t.wpg, t.tpw, t.pps = info.wpg, info.tpw, info.pps

    @property
    def function_name(self) -> str:
        t = self._tune
        if t.engine == 2:
            return f"{self.kernel_name}__tcgen05"
        return f"{self.kernel_name}__wpg{t.wpg}_tpw{t.tpw}_pps{t.pps}"

    @property
    def source(self) -> str:
        from ..compiler.compile_kernel import kernel_source

        t = self._tune
        return kernel_source(self.function_name, self.kind == _clib.WGRAD, self.params.r, self.params.s,
                             t.wpg, t.tpw, t.pps, engine=2 if t.engine == 2 else 1)

    def compile(self, device_attr=None) -> None:
        from ..compiler import flags
        from ..compiler.compile_kernel import compile_kernel
        from ..cuda.driver import B200_ATTRIBUTES

        attr = device_attr or B200_ATTRIBUTES
        try:
            self._resolve_tune(attr)
            info = _clib.PlanInfo()
            _clib.check(_clib.load().spio_conv2d_gw8_plan_jit(
                self.kind, ctypes.byref(self._shape), self._tune_ref(), attr.multiprocessor_count,
                attr.max_shared_memory_per_block_optin, ctypes.byref(info)), self.kernel_name)
            self.plan = info.as_dict()
            self._arch = attr.compute_capability
            self.cubin, self.compile_log = compile_kernel(
                self.source, source_name=self.function_name + ".cu", arch=self._arch,
                debug=flags.debug.get(), lineinfo=flags.lineinfo.get(), return_log=True)
        except Exception as exc:
            raise ValueError(f"Error in kernel {self}: {exc}") from exc

    def load(self, device_ordinal: int = 0, clear_cubin: bool = True) -> None:
        from ..compiler.compile_kernel import load_kernel

        if not torch.cuda.is_available():
            raise ValueError("CUDA error: no CUDA device is available")
        if self.cubin is None:
            raise ValueError(f"Error in kernel {self}: compile() must be called before load()")
        self._lib = _clib.load()
        self._device_ordinal = device_ordinal
        self.module, self.function = load_kernel(self.function_name, self.cubin, device_ordinal)
        self._check_register_hand_over()
        self.function.set_max_dynamic_shared_memory_size(self.plan["smem_bytes"])
        if self.kind == _clib.WGRAD:
            self.dbias_function = self.module.get_function(self.function_name + "__dbias")
            self.dbias_function.set_max_dynamic_shared_memory_size(self.plan["smem_bytes"])
        self._scratch_bytes = int(self.plan["scratch_bytes"])
        if clear_cubin:
            self.cubin = None

    def _check_register_hand_over(self) -> None:
        """Forward kernels with two or three warps per group move registers from the producer
        warpgroup to the consumers (setmaxnreg); the move is sized for the register count ptxas
        allocates under the kernel's launch bound.  Refuse to launch a kernel that was allocated
        anything else: its consumers could wait for registers for ever."""
        t = self._tune
        if self.kind == _clib.WGRAD or t.engine == 2 or t.wpg < 2:
            return
        launch = self.function.get_attribute("num_regs")
        consumer = 112 if t.wpg == 2 else 80
        if launch > consumer or 8 * t.wpg * 32 * (consumer - launch) > 128 * (launch - 24):
            self.unload()
            raise ValueError(f"Error in kernel {self}: allocated {launch} registers per thread; "
                             f"the register hand-over of the forward kernel does not fit")

    @property
    def function_handle(self):
        return self.function.handle if self.function is not None else None

    @property
    def dbias_function_handle(self):
        return self.dbias_function.handle if self.dbias_function is not None else None

    def unload(self) -> None:
        self.function = None
        self.dbias_function = None
        if self.module is not None:
            self.module.unload()
            self.module = None
        super().unload()

    @property
    def resource_usage(self) -> dict:
        """Registers per thread, spill bytes and static shared memory of the loaded function."""
        if self.function is None:
            raise ValueError(f"Error in kernel {self}: kernel is not loaded")
        return {k: self.function.get_attribute(k) for k in ("num_regs", "local_size_bytes", "shared_size_bytes")}

    # ------------------------------------------------------------ launch
    def launch(self, *args) -> None:
        """Same argument lists as :meth:`Kernel.launch`.  The library plans the launch, encodes (and
        caches) the tensor maps and launches the function through cuLaunchKernelEx with the
        programmatic-dependent-launch attribute, exactly as it does for its built-in variants."""
        if self.function is None:
            raise ValueError(f"Error in kernel {self}: kernel is not loaded")
        try:
            self._args_checker(args)
            dev = args[0].device
            with torch.cuda.device(dev):
                stream = torch.cuda.current_stream(dev).cuda_stream
                ptr = [a.data_ptr() if a is not None else None for a in args]
                sh, tn, fn = ctypes.byref(self._shape), self._tune_ref(), self.function.handle
                if self.kind == _clib.FPROP:
                    rc = self._lib.spio_conv2d_gw8_fprop_jit(fn, ptr[0], ptr[1], ptr[2], ptr[3], sh, tn, stream)
                elif self.kind == _clib.DGRAD:
                    rc = self._lib.spio_conv2d_gw8_dgrad_jit(fn, ptr[0], ptr[1], ptr[2], sh, tn, stream)
                else:
                    from .kernel import scratch_for

                    scratch = scratch_for(dev, stream, self._scratch_bytes)
                    rc = self._lib.spio_conv2d_gw8_wgrad_jit(fn, ptr[0], ptr[1], ptr[2], sh, tn,
                                                             scratch.data_ptr(), self._scratch_bytes, stream)
                _clib.check(rc)
        except Exception as exc:
            raise ValueError(f"Error in kernel {self}: {exc}") from exc

    __call__ = launch

    @property
    def launch_params(self) -> Optional[LaunchParams]:
        if self.plan is None:
            return None
        return LaunchParams(self.plan["grid"], self.plan["threads"], self.plan["smem_bytes"])

    def __repr__(self) -> str:
        return f"{self.kernel_name} {self.config} (jit)"


__all__ = ["JitKernel", "KIND_BY_NAME"]
