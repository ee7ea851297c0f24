"""Device attributes the kernel planner and the configuration spaces depend on.

Counterpart of ``get_device_attributes`` in the reference's Cython driver module
(spio/cuda/driver.pyx:275-330); here the values come from the CUDA runtime through
torch, and a fixed B200 record is available for planning on machines without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache
from typing import Optional, Tuple


@dataclass(frozen=True)
class DeviceAttributes:
    name: str = "NVIDIA B200"
    multiprocessor_count: int = 148
    l2_cache_size: int = 132120576
    compute_capability: Tuple[int, int] = (10, 0)
    max_shared_memory_per_block_optin: int = 232448
    max_shared_memory_per_block: int = 49152
    num_partitions_per_sm: int = 4

    @property
    def arch(self) -> str:
        major, minor = self.compute_capability
        return f"sm_{major}{minor}" + ("a" if major >= 9 else "")


# What `get_device_attributes` returns on the B200s this package targets.
B200_ATTRIBUTES = DeviceAttributes()


@lru_cache(maxsize=None)
def get_device_attributes(device_ordinal: int = 0) -> DeviceAttributes:
    import torch

    if not torch.cuda.is_available():
        raise ValueError("CUDA error: no CUDA device is available")
    prop = torch.cuda.get_device_properties(device_ordinal)
    return DeviceAttributes(
        name=prop.name,
        multiprocessor_count=prop.multi_processor_count,
        l2_cache_size=getattr(prop, "L2_cache_size", 0),
        compute_capability=(prop.major, prop.minor),
        max_shared_memory_per_block_optin=getattr(prop, "shared_memory_per_block_optin", 232448),
        max_shared_memory_per_block=getattr(prop, "shared_memory_per_block", 49152),
        num_partitions_per_sm=4,
    )


class Function:
    """A ``__global__`` function of a loaded :class:`Module`.

    Counterpart of the reference's ``Function`` (spio/cuda/driver.pyx:126-208): ``launch``
    takes the grid, the block and the kernel arguments and marshals them for
    ``cuLaunchKernel``.  Differences: the launch goes to torch's current stream instead
    of the NULL stream, and besides tensors, ``None``, ints and floats, an argument may be
    a ctypes object (a structure passed by value, such as a tensor map).
    """

    ATTRIBUTES = {"num_regs": 0, "local_size_bytes": 1, "shared_size_bytes": 2, "max_threads_per_block": 3}

    def __init__(self, handle: int, name: str, module: "Module"):
        self._handle = handle
        self.name = name
        self._module = module  # keeps the module loaded while the function is in use

    def set_max_dynamic_shared_memory_size(self, size: int) -> None:
        from .. import _clib

        _clib.check(_clib.load().spio_function_set_max_dynamic_smem(self._handle, int(size)), self.name)

    def get_attribute(self, name: str) -> int:
        import ctypes

        from .. import _clib

        value = ctypes.c_int()
        _clib.check(_clib.load().spio_function_get_attribute(self._handle, self.ATTRIBUTES[name],
                                                             ctypes.byref(value)), self.name)
        return value.value

    @staticmethod
    def _marshal(arg):
        import ctypes

        import torch

        if arg is None:
            return ctypes.c_void_p(0)
        if isinstance(arg, torch.Tensor):
            if not arg.is_cuda:
                raise ValueError("kernel arguments must be CUDA tensors")
            return ctypes.c_void_p(arg.data_ptr())
        if isinstance(arg, bool):
            return ctypes.c_int(int(arg))
        if isinstance(arg, int):
            return ctypes.c_int(arg)
        if isinstance(arg, float):
            return ctypes.c_float(arg)
        if isinstance(arg, (ctypes.Structure, ctypes.Array, ctypes._SimpleCData)):
            return arg
        raise ValueError(f"unsupported kernel argument type {type(arg).__name__}")

    def launch(self, grid, block, args, shared_mem_bytes: int = 0, stream: Optional[int] = None,
               programmatic: bool = False) -> None:
        """``programmatic=True`` launches through cuLaunchKernelEx with the programmatic-stream-
        serialization attribute; only for kernels that execute ``griddepcontrol.wait`` before they
        touch memory written by their predecessor in the stream."""
        import ctypes

        import torch

        from .. import _clib

        grid_x = grid[0] if isinstance(grid, (tuple, list)) else grid
        block_x = block[0] if isinstance(block, (tuple, list)) else block
        if isinstance(grid, (tuple, list)) and any(d != 1 for d in grid[1:]) or \
                isinstance(block, (tuple, list)) and any(d != 1 for d in block[1:]):
            raise ValueError("only one-dimensional grids and blocks are supported")
        if len(args) > 16:
            raise ValueError("at most 16 kernel arguments are supported")
        values = [self._marshal(a) for a in args]
        pointers = (ctypes.c_void_p * max(len(values), 1))()
        for i, v in enumerate(values):
            pointers[i] = ctypes.addressof(v)
        if stream is None:
            stream = torch.cuda.current_stream().cuda_stream
        lib = _clib.load()
        if programmatic:
            _clib.check(lib.spio_function_launch_ex(self._handle, int(grid_x), int(block_x), int(shared_mem_bytes),
                                                    stream, pointers, 1), self.name)
        else:
            _clib.check(lib.spio_function_launch(self._handle, int(grid_x), int(block_x),
                                                 int(shared_mem_bytes), stream, pointers), self.name)

    @property
    def handle(self) -> int:
        """The CUfunction, as an integer, for the library's ``*_jit`` entry points."""
        return self._handle


class Module:
    """A cubin loaded into the current device's primary context
    (reference: spio/cuda/driver.pyx:210-273)."""

    def __init__(self):
        self._handle: Optional[int] = None

    def load_data(self, cubin: bytes) -> None:
        import ctypes

        from .. import _clib

        if self._handle is not None:
            raise ValueError("module is already loaded")
        handle = ctypes.c_void_p()
        _clib.check(_clib.load().spio_module_load(cubin, ctypes.byref(handle)), "module load")
        self._handle = handle.value

    def get_function(self, name: str) -> Function:
        import ctypes

        from .. import _clib

        if self._handle is None:
            raise ValueError("module is not loaded")
        fn = ctypes.c_void_p()
        _clib.check(_clib.load().spio_module_get_function(self._handle, name.encode(), ctypes.byref(fn)), name)
        return Function(fn.value, name, self)

    def unload(self) -> None:
        from .. import _clib

        if self._handle is not None:
            handle, self._handle = self._handle, None
            _clib.check(_clib.load().spio_module_unload(handle), "module unload")

    def __del__(self):
        try:
            self.unload()
        except Exception:
            pass
