"""Generators: Python specifications that emit the C++ types a kernel is written against.

Counterpart of the reference's ``spio.generators`` (generators.py:17-223, tensor.py:18-576,
compound_index.py:14-93, dim.py, fold.py), rebuilt on the compact typed-dimension headers in
``spio_b200/csrc/typed.h`` and extended with what sm_100a kernels are made of: tiled TMA tensor
maps with typed coordinates (:class:`TensorMapSpec`), shared-memory rings guarded by mbarriers
(:class:`MbarrierRing`) and the tile configuration of the gw8 kernels (:class:`TileConfig`); typed
matrix fragments of the warp-level MMA (:class:`Fragment`), named constants (:class:`ParamsSpec`) and
macros (:class:`Macro`) as the reference has them.

    g = Generators()
    g.C = Dim()
    g.C8 = Fold(g.C, 8)
    g.X = Tensor(dtype.half, Dims(n=4, h=8, w=8, c=64))
    g.ThreadIdx = CompoundIndex(Dims(warp=4, lane=32))
    header = generate(g)            # text of a header; hand it to compile_kernel(header_dict=...)
"""

from .specs import (BUILTIN_DIM_NAMES, CompoundIndex, Dim, Dims, Fold, Fragment, FragmentType, GenSpec, Generators,
                    Macro, MbarrierRing, ParamsSpec, Strides, Tensor, TensorMapSpec, TileConfig, dtype, extract_specs,
                    generate, generate_from_source)
from .gw8 import gw8_kernel_specs, gw8_translation_unit

GENERATORS = ["Dim", "Fold", "Tensor", "CompoundIndex", "TensorMapSpec", "MbarrierRing", "TileConfig", "Fragment",
              "ParamsSpec", "Macro"]

__all__ = GENERATORS + ["BUILTIN_DIM_NAMES", "Dims", "Strides", "FragmentType", "GenSpec", "Generators", "dtype", "generate",
                        "extract_specs", "generate_from_source", "gw8_kernel_specs", "gw8_translation_unit"]
