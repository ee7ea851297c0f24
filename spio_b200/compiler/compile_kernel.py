"""Compile one kernel just in time and load it on a device.

Counterpart of the reference's spio/compiler/compile_kernel.py:14-120.  The reference
compiles a source file of the package against a generated header of index types; here the
kernels are templates on a tile configuration (``Gw8Config<R, S, WPG, TPW, PPS>``) and the
translation unit that instantiates one of them is generated: the kernel headers plus an
``extern "C"`` ``__global__`` wrapper whose name carries the layer parameters.
"""

from __future__ import annotations

from typing import Dict, Optional, Tuple

from .compile import compile_cuda
from .cuda_paths import kernel_headers

FORWARD_SOURCE = """\
#include "conv2d_gw8_fwd.cuh"
using namespace spio_b200;
using Cfg = Gw8Config<{r}, {s}, {wpg}, {tiles}, {pps}>;
extern "C" __global__ void __launch_bounds__(Cfg::THREADS, 1)
{name}(const __grid_constant__ TensorMap in_map, const __grid_constant__ TensorMap out_map,
       const Gw8Geom g, const __half* __restrict__ wgt, const float* __restrict__ bias, int ns, int nob,
       int* __restrict__ status) {{
  conv2d_gw8_fwd_body<Cfg>(in_map, out_map, g, wgt, bias, ns, nob, status);
}}
"""

TC_SOURCE = """\
#include "conv2d_gw8_fwd_tc.cuh"
using namespace spio_b200;
using Cfg = Gw8TcConfig<{r}, {s}>;
extern "C" __global__ void __launch_bounds__(Cfg::THREADS, 1)
{name}(const __grid_constant__ TensorMap in_map, const __grid_constant__ TensorMap row_map,
       const __grid_constant__ TensorMap out_map, const Gw8Geom g, const __half* __restrict__ wgt,
       const float* __restrict__ bias, int ns, int nob, int* __restrict__ status) {{
  conv2d_gw8_fwd_tc_body<Cfg>(in_map, row_map, out_map, g, wgt, bias, ns, nob, status);
}}
"""

WGRAD_SOURCE = """\
#include "conv2d_gw8_wgrad.cuh"
using namespace spio_b200;
using Cfg = Gw8Config<{r}, {s}, {wpg}, {tiles}, {pps}>;
extern "C" __global__ void __launch_bounds__(Cfg::WGRAD_THREADS, 1)
{name}(const __grid_constant__ TensorMap x_map, const __grid_constant__ TensorMap dy_map, const Gw8Geom g,
       float* __restrict__ scratch, int ns, int* __restrict__ status) {{
  conv2d_gw8_wgrad_body<Cfg>(x_map, dy_map, g, scratch, ns, status);
}}
// the instantiation that also sums dy for the bias gradient (odd number of filter taps)
extern "C" __global__ void __launch_bounds__(Cfg::WGRAD_THREADS, 1)
{name}__dbias(const __grid_constant__ TensorMap x_map, const __grid_constant__ TensorMap dy_map, const Gw8Geom g,
       float* __restrict__ scratch, int ns, int* __restrict__ status) {{
  conv2d_gw8_wgrad_body<Cfg, true>(x_map, dy_map, g, scratch, ns, status);
}}
"""


def kernel_source(kernel_name: str, wgrad: bool, r: int, s: int, wpg: int, tpw: int, pps: int,
                  engine: int = 1) -> str:
    """Source text of the translation unit for one kernel.

    ``tpw`` counts 8-pixel tiles per warp.  The weight-gradient kernel is instantiated
    with it directly; the forward kernel works on 16-pixel blocks and takes
    ``ceil(tpw / 2)`` of them per warp, as the variants built into the library do.
    """
    if not kernel_name.isidentifier():
        raise ValueError(f"{kernel_name!r} is not a valid kernel name")
    if engine == 2:
        if wgrad or r > 3 or s > 3:
            raise ValueError("the tcgen05 kernel computes fprop and dgrad for filters up to 3 x 3")
        return TC_SOURCE.format(name=kernel_name, r=r, s=s)
    if wgrad:
        return WGRAD_SOURCE.format(name=kernel_name, r=r, s=s, wpg=wpg, tiles=tpw, pps=pps)
    return FORWARD_SOURCE.format(name=kernel_name, r=r, s=s, wpg=wpg, tiles=(tpw + 1) // 2, pps=pps)


def compile_kernel(
    source: str,
    source_name: str = "kernel.cu",
    header_dict: Optional[Dict[str, str]] = None,
    arch: Tuple[int, int] = None,
    debug: bool = False,
    lineinfo: bool = False,
    max_registers: Optional[int] = None,
    return_log: bool = False,
    defines: Optional[Dict[str, object]] = None,
):
    """Compile kernel source text against the package's kernel headers; returns the cubin.
    ``defines`` become ``-D`` options (for instance ``SPIO_WAIT_LIMIT_NS``, the bound of the
    kernels' barrier waits)."""
    assert arch is not None, "Must specify GPU architecture for kernel compilation."
    if isinstance(arch, tuple) and arch[0] < 10:
        raise ValueError("Minimum supported GPU compute capability is sm_100a (Blackwell B200).")
    headers = kernel_headers()
    headers.update(header_dict or {})
    return compile_cuda(source, arch=arch, device_debug=debug, lineinfo=lineinfo, header_dict=headers,
                        max_registers=max_registers, src_name=source_name, ptxas_verbose=return_log,
                        default_device=True,  # the kernels' generic lambdas carry no __device__ mark
                        return_log=return_log, defines=defines)


def load_kernel(kernel_name: str, cubin: bytes, device_ordinal: int = 0):
    """(Module, Function) of a compiled kernel on a device."""
    import torch

    from ..cuda.driver import Module

    with torch.cuda.device(device_ordinal):
        torch.cuda.current_stream()  # makes the primary context current
        module = Module()
        module.load_data(cubin)
        return module, module.get_function(kernel_name)


def compile_and_load_kernel(kernel_name: str, source: str, device_ordinal: int = 0, arch=None, **kwargs):
    if arch is None:
        from ..cuda.driver import get_device_attributes

        arch = get_device_attributes(device_ordinal).compute_capability
    cubin = compile_kernel(source, source_name=kernel_name + ".cu", arch=arch, **kwargs)
    return load_kernel(kernel_name, cubin, device_ordinal)
