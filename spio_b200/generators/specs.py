"""Generator specifications and the code they emit.

Every specification knows its C++ type name (given by the :class:`Generators` container or
passed explicitly), the specifications it depends on, and the one declaration it contributes
to the generated header.  :func:`generate` orders the declarations so that every type is
declared before it is used and declares dimensions that are only mentioned by name.
"""

from __future__ import annotations

import re
import textwrap
from enum import Enum
from typing import Dict, Iterable, Iterator, List, Optional, Sequence, Tuple, Union

NAMESPACE = "spio_b200::typed"

# Dimension names the headers give a meaning of their own (the reference reserves LANE and
# OFFSET the same way, spio/generators/dim.py).
BUILTIN_DIM_NAMES = ("LANE", "OFFSET")


class dtype(Enum):
    """Element types of tensors and tensor maps: (C++ name, bytes)."""

    float = ("float", 4)
    float2 = ("float2", 8)
    float4 = ("float4", 16)
    half = ("__half", 2)
    half2 = ("__half2", 4)
    uint = ("unsigned", 4)
    uint2 = ("uint2", 8)
    uint4 = ("uint4", 16)
    int32 = ("int", 4)

    @property
    def cname(self) -> str:
        return self.value[0]

    @property
    def nbytes(self) -> int:
        return self.value[1]


_FOLD_NAME = re.compile(r"^([A-Za-z_]+?)(\d+)$")


def split_fold_name(name: str) -> Tuple[str, Optional[int]]:
    """``"C8"`` -> ``("C", 8)``; ``"C"`` -> ``("C", None)``."""
    m = _FOLD_NAME.match(name)
    if m is None:
        return name, None
    return m.group(1), int(m.group(2))


class GenSpec:
    """Base of all specifications."""

    class_name: Optional[str] = None

    def _set_class_name(self, name: str):
        if self.class_name not in (None, name):
            raise ValueError(f"specification is already named {self.class_name!r}, cannot rename it {name!r}")
        self.class_name = name
        return None

    def used(self) -> List["GenSpec"]:
        return []

    def declaration(self) -> str:
        raise NotImplementedError

    def _need_name(self) -> str:
        if self.class_name is None:
            raise ValueError(f"{type(self).__name__} has no name: assign it to a Generators attribute or pass name=")
        return self.class_name


class Dim(GenSpec):
    """A named dimension: ``struct I_tag; using I = Dim<I_tag>;``.  Calling a dimension gives a
    sized one for use in :class:`Dims`: ``Dims(g.I(16), g.K(32))``."""

    def __init__(self, name: Optional[str] = None):
        self.class_name = name.upper() if name else None

    def _set_class_name(self, name: str):
        return super()._set_class_name(name)

    def __call__(self, size: int) -> Tuple["Dim", int]:
        return (self, int(size))

    def fold(self, stride: int, name: Optional[str] = None) -> "Fold":
        return Fold(self, stride, name=name)

    def declaration(self) -> str:
        n = self._need_name()
        return f"struct {n}_tag;\nusing {n} = {NAMESPACE}::Dim<{n}_tag>;"

    def __eq__(self, other):
        return isinstance(other, Dim) and self.class_name is not None and self.class_name == other.class_name

    def __hash__(self):
        return hash(("Dim", self.class_name)) if self.class_name else id(self)

    def __repr__(self):
        return f"Dim({self.class_name})"


class Fold(GenSpec):
    """A dimension counted in blocks of ``stride``: ``using C8 = Fold<C, 8>;``.  ``dim`` is a
    :class:`Dim`, another :class:`Fold` (folds compose) or a dimension name."""

    def __init__(self, dim: Union[Dim, "Fold", str], stride: int, name: Optional[str] = None):
        if int(stride) <= 0:
            raise ValueError("fold stride must be positive")
        self.dim = Dim(dim) if isinstance(dim, str) else dim
        self.stride = int(stride)
        self.class_name = name

    def __call__(self, size: int) -> Tuple["Fold", int]:
        return (self, int(size))

    @property
    def base(self) -> Dim:
        return self.dim.base if isinstance(self.dim, Fold) else self.dim

    @property
    def total_stride(self) -> int:
        return self.stride * (self.dim.total_stride if isinstance(self.dim, Fold) else 1)

    def used(self) -> List[GenSpec]:
        return [self.dim]

    def declaration(self) -> str:
        return f"using {self._need_name()} = {NAMESPACE}::Fold<{self.dim._need_name()}, {self.stride}>;"

    def __repr__(self):
        return f"Fold({self.dim!r}, {self.stride})"


DimLike = Union[Dim, Fold]


def _dim_from_name(name: str) -> DimLike:
    """``"c"`` -> Dim C; ``"c8"`` -> Fold(C, 8) named C8 (an implicit fold, as in the reference)."""
    upper = name.upper()
    base, stride = split_fold_name(upper)
    if stride is None:
        return Dim(upper)
    return Fold(Dim(base), stride, name=upper)


class Dims:
    """An ordered list of sized dimensions, outermost first: ``Dims(n=4, h=8, c8=8, c=8)`` by
    name (a trailing number makes a fold), or ``Dims(g.I(16), g.K(32))`` with declared ones."""

    def __init__(self, *sized: Tuple[DimLike, int], **named: int):
        self.items: List[Tuple[DimLike, int]] = []
        for entry in sized:
            if not (isinstance(entry, tuple) and len(entry) == 2 and isinstance(entry[0], (Dim, Fold))):
                raise TypeError("positional entries of Dims are sized dimensions such as I(16)")
            self.items.append((entry[0], int(entry[1])))
        for name, size in named.items():
            self.items.append((_dim_from_name(name), int(size)))
        if not self.items:
            raise ValueError("Dims needs at least one dimension")
        for _, size in self.items:
            if size <= 0:
                raise ValueError("dimension sizes must be positive")

    def __iter__(self) -> Iterator[Tuple[DimLike, int]]:
        return iter(self.items)

    def __len__(self) -> int:
        return len(self.items)

    @property
    def sizes(self) -> List[int]:
        return [s for _, s in self.items]

    @property
    def total(self) -> int:
        n = 1
        for s in self.sizes:
            n *= s
        return n

    def row_major_strides(self) -> List[int]:
        strides, acc = [], 1
        for s in reversed(self.sizes):
            strides.append(acc)
            acc *= s
        return strides[::-1]


class Strides:
    """Explicit element strides by dimension name for a :class:`Tensor` (others stay row-major)."""

    def __init__(self, **named: int):
        self.named = {k.upper(): int(v) for k, v in named.items()}


class Tensor(GenSpec):
    """A pointer with compile-time sizes and strides:
    ``using X = Tensor<T, Extent<N, 4, 4096>, ...>;``"""

    def __init__(self, data_type: dtype, dims: Dims, strides: Optional[Strides] = None, constant: bool = False,
                 name: Optional[str] = None):
        self.data_type = data_type
        self.dims = dims
        self.constant = bool(constant)
        self.class_name = name
        self.strides = dims.row_major_strides()
        if strides is not None:
            # an explicit stride also moves the strides of the dimensions outside it
            names = [d._need_name() for d, _ in dims]
            unknown = set(strides.named) - set(names)
            if unknown:
                raise ValueError(f"Strides names dimensions the tensor does not have: {sorted(unknown)}")
            acc = 1
            for i in range(len(dims) - 1, -1, -1):
                if names[i] in strides.named:
                    if strides.named[names[i]] < acc:
                        raise ValueError(f"stride of {names[i]} overlaps the dimensions inside it")
                    acc = strides.named[names[i]]
                self.strides[i] = acc
                acc *= dims.sizes[i]

    def used(self) -> List[GenSpec]:
        return [d for d, _ in self.dims]

    @property
    def storage_size(self) -> int:
        return 1 + sum((size - 1) * stride for (_, size), stride in zip(self.dims, self.strides))

    def declaration(self) -> str:
        t = ("const " if self.constant else "") + self.data_type.cname
        extents = ", ".join(f"{NAMESPACE}::Extent<{d._need_name()}, {size}, {stride}>"
                            for (d, size), stride in zip(self.dims, self.strides))
        return f"using {self._need_name()} = {NAMESPACE}::Tensor<{t}, {extents}>;"


class CompoundIndex(GenSpec):
    """Splits a linear offset into typed indices, first dimension slowest:
    ``using ThreadIdx = CompoundIndex<Extent<WARP, 4, 0>, Extent<LANE, 32, 0>>;``"""

    def __init__(self, dims: Dims, name: Optional[str] = None):
        self.dims = dims
        self.class_name = name

    def used(self) -> List[GenSpec]:
        return [d for d, _ in self.dims]

    @property
    def size(self) -> int:
        return self.dims.total

    def declaration(self) -> str:
        extents = ", ".join(f"{NAMESPACE}::Extent<{d._need_name()}, {size}, 0>" for d, size in self.dims)
        return f"using {self._need_name()} = {NAMESPACE}::CompoundIndex<{extents}>;"


class TensorMapSpec(GenSpec):
    """A tiled TMA tensor map with typed coordinates.

    ``box`` lists the axes INNERMOST FIRST with the box size along each (1 to 4 axes; missing
    outer axes get a box of one).  The innermost box must be a whole number of 16 bytes and, with
    a swizzle, no wider than the swizzle span.  ``encode_args(tensor_sizes)`` gives the arguments
    of the library's ``spio_tensor_map_encode`` for a tensor of the given extents."""

    SWIZZLE = {0: 0, 32: 1, 64: 2, 128: 3}

    def __init__(self, data_type: dtype, box: Dims, swizzle: int = 128, name: Optional[str] = None):
        if not 1 <= len(box) <= 4:
            raise ValueError("a tiled tensor map has 1 to 4 axes")
        if swizzle not in self.SWIZZLE:
            raise ValueError("swizzle must be 0, 32, 64 or 128 bytes")
        inner = box.sizes[0] * data_type.nbytes
        if inner % 16:
            raise ValueError("the innermost box extent must be a whole number of 16 bytes")
        if swizzle and inner > swizzle:
            raise ValueError("the innermost box extent must not exceed the swizzle span")
        if any(s > 256 for s in box.sizes):
            raise ValueError("box extents are at most 256")
        self.data_type = data_type
        self.box = box
        self.swizzle = swizzle
        self.class_name = name

    def used(self) -> List[GenSpec]:
        return [d for d, _ in self.box]

    @property
    def box_bytes(self) -> int:
        return self.box.total * self.data_type.nbytes

    def declaration(self) -> str:
        items = list(self.box)
        extents = [f"{NAMESPACE}::Extent<{d._need_name()}, {size}, 0>" for d, size in items]
        while len(extents) < 4:  # unused outer axes: a box of one along a dimension nothing indexes
            extents.append(f"{NAMESPACE}::Extent<{NAMESPACE}::Dim<void>, 1, 0>")
        return (f"using {self._need_name()} = {NAMESPACE}::TensorMapRef<{self.data_type.cname}, "
                + ", ".join(extents) + ">;")

    def encode_args(self, sizes: Sequence[int], strides_bytes: Optional[Sequence[int]] = None) -> Dict[str, object]:
        """Sizes (and optionally byte strides of axes 1..) of the tensor, innermost first."""
        rank = len(self.box)
        if len(sizes) != rank:
            raise ValueError(f"the map has {rank} axes")
        if strides_bytes is None:
            strides_bytes, acc = [], self.data_type.nbytes
            for s in sizes[:-1]:
                acc *= s
                strides_bytes.append(acc)
        if any(s % 16 for s in strides_bytes):
            raise ValueError("tensor strides must be multiples of 16 bytes")
        pad = 4 - rank
        return {"elem_bytes": self.data_type.nbytes, "rank": 4,
                "sizes": list(sizes) + [1] * pad,
                "strides_bytes": list(strides_bytes) + [strides_bytes[-1] * sizes[-1] if strides_bytes else
                                                        sizes[0] * self.data_type.nbytes] * pad,
                "box": self.box.sizes + [1] * pad, "swizzle": self.SWIZZLE[self.swizzle]}


class MbarrierRing(GenSpec):
    """A producer / consumer ring of shared-memory slots: ``using Ring = MbarrierRing<4>;``"""

    def __init__(self, slots: int, name: Optional[str] = None):
        if not 1 <= int(slots) <= 32:
            raise ValueError("a ring has 1 to 32 slots")
        self.slots = int(slots)
        self.class_name = name

    def declaration(self) -> str:
        return f"using {self._need_name()} = {NAMESPACE}::MbarrierRing<{self.slots}>;"


class TileConfig(GenSpec):
    """Compile-time tile configuration of the gw8 kernels:
    ``using Cfg = spio_b200::Gw8Config<R, S, WPG, TILES, PPS>;`` (filter size, compute warps per
    channel group, tiles per warp, row pairs per ring slot)."""

    def __init__(self, r: int, s: int, wpg: int, tiles: int, pps: int, name: Optional[str] = None):
        if not (1 <= r <= 5 and 1 <= s <= 5):
            raise ValueError("filter extents are 1 to 5")
        if not (1 <= wpg <= 3 and 1 <= tiles <= 8 and 1 <= pps <= 4):
            raise ValueError("wpg is 1..3, tiles 1..8, pps 1..4")
        self.r, self.s, self.wpg, self.tiles, self.pps = int(r), int(s), int(wpg), int(tiles), int(pps)
        self.class_name = name

    def declaration(self) -> str:
        return (f"using {self._need_name()} = spio_b200::Gw8Config<{self.r}, {self.s}, {self.wpg}, "
                f"{self.tiles}, {self.pps}>;")


class FragmentType(Enum):
    """Warp-level MMA fragments (fp16 x fp16 -> fp32), named as in the reference
    (spio/generators/fragment_type.py): (C++ template, what its two dimensions are)."""

    M16_N8_F32_C = ("MmaM16N8F32C", ("row", "col"))
    M16_K16_F16_A = ("MmaM16K16F16A", ("row", "k"))
    N8_K16_F16_B = ("MmaN8K16F16B", ("col", "k"))
    M16_K8_F16_A = ("MmaM16K8F16A", ("row", "k"))
    N8_K8_F16_B = ("MmaN8K8F16B", ("col", "k"))


class Fragment(GenSpec):
    """A matrix fragment whose rows / columns / k are typed dimensions:
    ``using Acc = MmaM16N8F32C<I, J>;``.  ``first`` and ``second`` are the two dimensions in the
    order the fragment type names them (C: row, column; A: row, k; B: column, k)."""

    def __init__(self, fragment_type: FragmentType, first: "DimLike", second: "DimLike", name: Optional[str] = None):
        if not isinstance(fragment_type, FragmentType):
            raise ValueError("fragment_type must be a FragmentType")
        self.fragment_type = fragment_type
        self.first = _dim_from_name(first) if isinstance(first, str) else first
        self.second = _dim_from_name(second) if isinstance(second, str) else second
        self.class_name = name

    def used(self) -> List[GenSpec]:
        return [self.first, self.second]

    def declaration(self) -> str:
        return (f"using {self._need_name()} = {NAMESPACE}::{self.fragment_type.value[0]}<"
                f"{self.first._need_name()}, {self.second._need_name()}>;")


class ParamsSpec(GenSpec):
    """Named compile-time constants: ``namespace Block { inline constexpr int p = 16; ... }``
    (bool, int or float values; the reference's ParamsSpec, spio/generators/params.py)."""

    def __init__(self, params: Dict[str, object], name: Optional[str] = None):
        for key, val in params.items():
            if not key.isidentifier():
                raise ValueError(f"{key!r} is not a C++ identifier")
            if not isinstance(val, (bool, int, float)):
                raise ValueError(f"parameter {key} has unsupported type {type(val).__name__}")
        self.params = dict(params)
        self.class_name = name

    def declaration(self) -> str:
        lines = [f"namespace {self._need_name()} {{"]
        for key, val in self.params.items():
            if isinstance(val, bool):
                lines.append(f"inline constexpr bool {key} = {'true' if val else 'false'};")
            elif isinstance(val, int):
                lines.append(f"inline constexpr int {key} = {val};")
            else:
                lines.append(f"inline constexpr float {key} = {val!r}f;")
        lines.append("}")
        return "\n".join(lines)


class Macro(GenSpec):
    """Preprocessor definitions: ``#define NAME value`` (the reference's Macro,
    spio/generators/macros.py).  Macros have no type name; a container names them only to keep
    them apart."""

    def __init__(self, macros: Dict[str, object], name: Optional[str] = None):
        for key in macros:
            if not key.isidentifier():
                raise ValueError(f"{key!r} is not a macro name")
        self.macros = dict(macros)
        self.class_name = name

    def _need_name(self) -> str:
        return self.class_name or "macros_" + "_".join(self.macros)

    def declaration(self) -> str:
        return "\n".join(f"#define {key} {val}" for key, val in self.macros.items())


class Generators:
    """Collects specifications; the attribute name becomes the C++ type name (the reference's
    container works the same way, spio/generators/generators_class.py:17-97)."""

    def __init__(self):
        object.__setattr__(self, "_registry", {})

    def __setattr__(self, name: str, value) -> None:
        if name.startswith("_") or not isinstance(value, GenSpec):
            object.__setattr__(self, name, value)
            return
        value._set_class_name(name)
        self._registry[name] = value

    def __getattr__(self, name: str):
        registry = object.__getattribute__(self, "_registry")
        if name in registry:
            return registry[name]
        raise AttributeError(f"'Generators' has no attribute '{name}'")

    def __iter__(self) -> Iterator[GenSpec]:
        return iter(self._registry.values())

    def __len__(self) -> int:
        return len(self._registry)

    def __contains__(self, name: str) -> bool:
        return name in self._registry

    def keys(self):
        return self._registry.keys()

    def items(self):
        return self._registry.items()

    def values(self):
        return self._registry.values()


def _ordered(specs: Iterable[GenSpec]) -> List[GenSpec]:
    """Dependencies first, each type once (two specifications of one name must agree)."""
    out: List[GenSpec] = []
    seen: Dict[str, str] = {}

    def visit(spec: GenSpec):
        for dep in spec.used():
            visit(dep)
        name = spec._need_name()
        text = spec.declaration()
        if name in seen:
            if seen[name] != text:
                raise ValueError(f"two different specifications are named {name}")
            return
        seen[name] = text
        out.append(spec)

    for spec in specs:
        visit(spec)
    return out


def generate(specs: Iterable[GenSpec], namespace: Optional[str] = None, tma: Optional[bool] = None) -> str:
    """Text of a header that declares every specification (and the dimensions they mention).
    ``tma`` forces or suppresses the include of the TMA / mbarrier wrappers; by default it is
    included when a :class:`TensorMapSpec`, :class:`MbarrierRing` or :class:`TileConfig` is present."""
    ordered = _ordered(list(specs))
    if tma is None:
        tma = any(isinstance(s, (TensorMapSpec, MbarrierRing, TileConfig)) for s in ordered)
    lines = ["#pragma once"]
    if any(getattr(s, "data_type", None) in (dtype.half, dtype.half2) for s in ordered):
        lines.append("#include <cuda_fp16.h>")
    lines.append('#include "typed_tma.cuh"' if tma else '#include "typed.h"')
    if any(isinstance(s, Fragment) for s in ordered):
        lines.append('#include "typed_mma.cuh"')
    if any(isinstance(s, TileConfig) for s in ordered):
        lines.append('#include "gw8_common.cuh"')
    lines.append("")
    if namespace:
        lines.append(f"namespace {namespace} {{")
    lines += [s.declaration() for s in ordered]
    if namespace:
        lines.append(f"}}  // namespace {namespace}")
    return "\n".join(lines) + "\n"


SPIO_BLOCK = re.compile(r"/\*@spio[ \t]*\n?(.*?)@spio\*/", re.DOTALL)


def extract_specs(source: str) -> Generators:
    """Specifications embedded in a CUDA / C++ source as ``/*@spio ... @spio*/`` comment blocks
    (the reference's tutorial sources carry theirs the same way, tests/test_tutorial.py:47).  The
    blocks are Python assignments, evaluated with the generator classes in scope and nothing else;
    each assigned name becomes a type name."""
    g = Generators()
    scope = {"__builtins__": {}, "dtype": dtype, "Dims": Dims, "Strides": Strides, "Dim": Dim, "Fold": Fold,
             "Tensor": Tensor, "CompoundIndex": CompoundIndex, "TensorMapSpec": TensorMapSpec,
             "MbarrierRing": MbarrierRing, "TileConfig": TileConfig, "Fragment": Fragment,
             "FragmentType": FragmentType, "ParamsSpec": ParamsSpec, "Macro": Macro, "dict": dict}
    class Naming(dict):
        """Block-level names: a specification is named the moment it is assigned, so that later
        lines of the same block can use it (``I = Dim()`` then ``Dims(I(16))``)."""

        def __setitem__(self, name, value):
            if isinstance(value, GenSpec):
                setattr(g, name, value)
            super().__setitem__(name, value)

    names = Naming()
    for block in SPIO_BLOCK.findall(source):
        exec(textwrap.dedent(block), scope, names)  # noqa: S102 - no builtins, generator classes only
    return g


def generate_from_source(source: str, namespace: Optional[str] = None) -> str:
    """Header for the ``/*@spio ... @spio*/`` blocks of ``source``."""
    return generate(extract_specs(source), namespace=namespace)
