"""A kernel written against generated typed-dimension types, run on the GPU.

spio_b200/examples/typed_tile_copy.cu carries its type specifications in @spio blocks; the test
generates the header, compiles the kernel with NVRTC, encodes the tiled tensor map through the C
ABI and checks that the copy is exact -- TMA load with typed coordinates, mbarrier ring, typed
tensor subscripting and compound indices all take part.
"""

import ctypes
from pathlib import Path

import pytest
import torch

from spio_b200 import _clib
from spio_b200.compiler import compile_kernel, load_kernel
from spio_b200.cuda import get_device_attributes
from spio_b200.generators import extract_specs, generate
from tests import capi

pytestmark = pytest.mark.gpu

SOURCE = Path(__file__).resolve().parent.parent / "spio_b200" / "examples" / "typed_tile_copy.cu"


def test_typed_tile_copy_kernel():
    src = SOURCE.read_text()
    specs = extract_specs(src)
    cubin = compile_kernel(src, source_name="typed_tile_copy.cu", header_dict={"types.h": generate(specs)},
                           arch=get_device_attributes(0).compute_capability)
    module, fn = load_kernel("typed_tile_copy", cubin, 0)
    lib = _clib.load()

    x = torch.randn(3, 8, 16, 64, device="cuda:0").half()            # N, H, W, C
    y = torch.full_like(x, capi.DEAD_VALUE)
    args = specs.XMap.encode_args([64, 16, 8, 3])                    # innermost first
    tmap = (ctypes.c_ulonglong * 16)()
    _clib.check(lib.spio_tensor_map_encode(
        tmap, x.data_ptr(), args["elem_bytes"], args["rank"], (ctypes.c_ulonglong * 4)(*args["sizes"]),
        (ctypes.c_ulonglong * 3)(*args["strides_bytes"]), (ctypes.c_uint * 4)(*args["box"]), args["swizzle"]))
    status = ctypes.c_void_p()
    _clib.check(lib.spio_b200_status_address(ctypes.byref(status)))
    fn.launch(specs.Block.size, 128, [tmap, y, status])
    torch.cuda.synchronize()
    assert capi.status() == 0
    assert torch.equal(x, y)
    module.unload()


def test_tensor_map_encode_rejects_bad_arguments():
    lib = _clib.load()
    x = torch.zeros(4096, dtype=torch.float16, device="cuda:0")
    tmap = (ctypes.c_ulonglong * 16)()
    sizes, strides, box = (ctypes.c_ulonglong * 2)(64, 32), (ctypes.c_ulonglong * 1)(128), (ctypes.c_uint * 2)(64, 8)
    _clib.check(lib.spio_tensor_map_encode(tmap, x.data_ptr(), 2, 2, sizes, strides, box, 3))
    assert lib.spio_tensor_map_encode(tmap, x.data_ptr() + 2, 2, 2, sizes, strides, box, 3) != 0
    assert "aligned" in _clib.last_error()
    assert lib.spio_tensor_map_encode(tmap, x.data_ptr(), 3, 2, sizes, strides, box, 3) != 0
    assert "element size" in _clib.last_error()
    bad_box = (ctypes.c_uint * 2)(4, 8)
    assert lib.spio_tensor_map_encode(tmap, x.data_ptr(), 2, 2, sizes, strides, bad_box, 0) != 0
    assert "16 bytes" in _clib.last_error()


def test_typed_mma_tile_kernel():
    """spio_b200/examples/typed_mma_tile.cu: typed fragments loaded with ldmatrix from typed
    shared-memory tensors, multiplied with the warp-level MMA and stored through their typed lane
    coordinates, against an fp32 matrix product of the same fp16 operands."""
    source = SOURCE.parent / "typed_mma_tile.cu"
    src = source.read_text()
    specs = extract_specs(src)
    cubin = compile_kernel(src, source_name="typed_mma_tile.cu", header_dict={"types.h": generate(specs)},
                           arch=get_device_attributes(0).compute_capability)
    module, fn = load_kernel("typed_mma_tile", cubin, 0)
    m, n, k = (specs.Shape.params[key] for key in ("m", "n", "k"))
    gen = torch.Generator(device="cuda:0").manual_seed(3)
    a = torch.randn(m, k, device="cuda:0", generator=gen).half()
    b = torch.randn(n, k, device="cuda:0", generator=gen).half()          # k contiguous: B is stored column by column
    c = torch.full((m, n), capi.DEAD_VALUE, dtype=torch.float32, device="cuda:0")
    fn.launch(specs.Tiles.size, 32, [a, b, c])
    torch.cuda.synchronize()
    ref = a.double() @ b.double().t()
    # fp32 accumulation over k = 96 products of fp16 values
    assert float((c.double() - ref).abs().max()) <= 1e-4 * float(ref.abs().max())
    module.unload()
