"""The gw8 kernels expressed through the generators: the translation unit the just-in-time path
compiles is the generated type header plus an ``extern "C"`` entry point per kernel.

The reference generates a ``types.h`` of index types per (layer shape, configuration) and
compiles the fixed kernel source against it (spio/kernels/conv2d_gw8_kernel.py:62-238).  Here the
layer shape is a run-time argument of the kernels, so the generated part is the tile
configuration and the typed views a kernel author needs of the operands.
"""

from __future__ import annotations

from .specs import Dims, Generators, MbarrierRing, TensorMapSpec, TileConfig, dtype, generate

FORWARD_ENTRY = """\
extern "C" __global__ void __launch_bounds__(Cfg::THREADS, 1)
{name}(const __grid_constant__ TensorMap in_map, const __grid_constant__ TensorMap out_map,
       const Gw8Geom g, const __half* __restrict__ wgt, const float* __restrict__ bias, int ns, int nob,
       int* __restrict__ status) {{
  conv2d_gw8_fwd_body<Cfg>(in_map, out_map, g, wgt, bias, ns, nob, status);
}}
"""

WGRAD_ENTRY = """\
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


def gw8_kernel_specs(r: int, s: int, wpg: int, tiles: int, pps: int, box_w: int = 64, nb: int = 1,
                     ring_slots: int = 4) -> Generators:
    """The specifications of one gw8 kernel instantiation: its tile configuration, the tensor
    maps of the streamed operand (a box of 64 channels x ``box_w`` pixels x 2 * pps rows x ``nb``
    images, 128-byte swizzle) and of a row pair of the tiled operand, and the slot ring."""
    g = Generators()
    g.Cfg = TileConfig(r, s, wpg, tiles, pps)
    g.StreamedMap = TensorMapSpec(dtype.half, Dims(c=64, w=box_w, h=2 * pps, n=nb))
    g.TiledMap = TensorMapSpec(dtype.half, Dims(c=64, w=max(box_w - 8 * ((s - 1 + 7) // 8), 8), h=2, n=nb))
    g.SlotRing = MbarrierRing(ring_slots)
    return g


def gw8_translation_unit(kernel_name: str, wgrad: bool, r: int, s: int, wpg: int, tiles: int, pps: int) -> str:
    """Source text handed to NVRTC: the kernel header, the generated tile configuration and the
    entry point(s)."""
    if not kernel_name.isidentifier():
        raise ValueError(f"{kernel_name!r} is not a valid kernel name")
    g = Generators()
    g.Cfg = TileConfig(r, s, wpg, tiles, pps)
    header = "conv2d_gw8_wgrad.cuh" if wgrad else "conv2d_gw8_fwd.cuh"
    types = "\n".join(line for line in generate(g, tma=False).splitlines() if not line.startswith("#"))
    entry = (WGRAD_ENTRY if wgrad else FORWARD_ENTRY).format(name=kernel_name)
    return f'#include "{header}"\nusing namespace spio_b200;\n{types.strip()}\n{entry}'
