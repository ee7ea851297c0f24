"""The generators: specifications -> C++ declarations, checked as text, by the host compiler and
by NVRTC.

Style of the reference's generator tests (tests/test_generators.py:238-290, tests/test_dims.py,
tests/test_tensor.py, tests/test_tutorial.py): the generated code is compared as strings, and the
typed headers are exercised by compiling and running small C++ programs.  Everything here runs
without a GPU; tests/test_generators_gpu.py runs a kernel written against generated types.
"""

import shutil
import subprocess
from pathlib import Path

import pytest

from spio_b200.compiler import compile_kernel
from spio_b200.compiler.compile_kernel import kernel_source
from spio_b200.generators import (CompoundIndex, Dim, Dims, Fold, Generators, MbarrierRing, Strides, Tensor,
                                  TensorMapSpec, TileConfig, dtype, extract_specs, generate, generate_from_source,
                                  gw8_kernel_specs, gw8_translation_unit)

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "spio_b200" / "csrc"
T = "spio_b200::typed"


def body(code: str):
    """Declaration lines of a generated header."""
    return [line for line in code.splitlines() if line and not line.startswith("#")]


class TestDeclarations:
    def test_dim_and_fold(self):
        g = Generators()
        g.C = Dim()
        g.C8 = Fold(g.C, 8)
        g.C64 = Fold(g.C8, 8)
        assert body(generate(g)) == [
            "struct C_tag;",
            f"using C = {T}::Dim<C_tag>;",
            f"using C8 = {T}::Fold<C, 8>;",
            f"using C64 = {T}::Fold<C8, 8>;",
        ]
        assert g.C64.total_stride == 64 and g.C64.base is g.C

    def test_tensor_row_major_by_name(self):
        g = Generators()
        g.X = Tensor(dtype.half, Dims(n=4, h=8, w=8, c=64), constant=True)
        code = generate(g)
        assert code.startswith('#pragma once\n#include <cuda_fp16.h>\n#include "typed.h"\n')
        assert body(code)[-1] == (
            f"using X = {T}::Tensor<const __half, {T}::Extent<N, 4, 4096>, {T}::Extent<H, 8, 512>, "
            f"{T}::Extent<W, 8, 64>, {T}::Extent<C, 64, 1>>;")
        # the dimensions the tensor mentions are declared once, before it
        assert body(code)[:2] == ["struct N_tag;", f"using N = {T}::Dim<N_tag>;"]
        assert g.X.storage_size == 4 * 8 * 8 * 64

    def test_tensor_with_implicit_fold_and_padded_stride(self):
        g = Generators()
        g.Smem = Tensor(dtype.uint4, Dims(w=18, c8=8), Strides(w=9))
        lines = body(generate(g))
        assert f"using C8 = {T}::Fold<C, 8>;" in lines
        assert lines[-1] == f"using Smem = {T}::Tensor<uint4, {T}::Extent<W, 18, 9>, {T}::Extent<C8, 8, 1>>;"
        assert g.Smem.storage_size == 17 * 9 + 7 + 1

    def test_tensor_with_declared_dims(self):
        g = Generators()
        g.I = Dim()
        g.K = Dim()
        g.A = Tensor(dtype.float, Dims(g.I(16), g.K(32)))
        assert body(generate(g))[-1] == f"using A = {T}::Tensor<float, {T}::Extent<I, 16, 32>, {T}::Extent<K, 32, 1>>;"

    def test_compound_index(self):
        g = Generators()
        g.ThreadIdx = CompoundIndex(Dims(warp=4, lane=32))
        assert g.ThreadIdx.size == 128
        assert body(generate(g))[-1] == (
            f"using ThreadIdx = {T}::CompoundIndex<{T}::Extent<WARP, 4, 0>, {T}::Extent<LANE, 32, 0>>;")

    def test_tensor_map_and_ring(self):
        g = Generators()
        g.XMap = TensorMapSpec(dtype.half, Dims(c=64, w=64, h=4, n=1))
        g.Rows = TensorMapSpec(dtype.half, Dims(c=64, w=16), swizzle=0)
        g.Ring = MbarrierRing(4)
        code = generate(g)
        assert '#include "typed_tma.cuh"' in code
        lines = body(code)
        assert (f"using XMap = {T}::TensorMapRef<__half, {T}::Extent<C, 64, 0>, {T}::Extent<W, 64, 0>, "
                f"{T}::Extent<H, 4, 0>, {T}::Extent<N, 1, 0>>;") in lines
        # missing outer axes become boxes of one along a dimension nothing indexes
        assert (f"using Rows = {T}::TensorMapRef<__half, {T}::Extent<C, 64, 0>, {T}::Extent<W, 16, 0>, "
                f"{T}::Extent<{T}::Dim<void>, 1, 0>, {T}::Extent<{T}::Dim<void>, 1, 0>>;") in lines
        assert lines[-1] == f"using Ring = {T}::MbarrierRing<4>;"
        assert g.XMap.box_bytes == 64 * 64 * 4 * 2

    def test_tensor_map_encode_arguments(self):
        m = TensorMapSpec(dtype.half, Dims(c=64, w=16, h=4, n=1), swizzle=0)
        args = m.encode_args([64, 16, 8, 3])
        assert args == {"elem_bytes": 2, "rank": 4, "sizes": [64, 16, 8, 3], "strides_bytes": [128, 2048, 16384],
                        "box": [64, 16, 4, 1], "swizzle": 0}

    def test_tile_config(self):
        g = Generators()
        g.Cfg = TileConfig(3, 3, 2, 2, 2)
        code = generate(g)
        assert '#include "gw8_common.cuh"' in code
        assert body(code) == ["using Cfg = spio_b200::Gw8Config<3, 3, 2, 2, 2>;"]

    def test_namespace_and_order(self):
        g = Generators()
        g.First = Tensor(dtype.float, Dims(i=1))
        g.Second = Tensor(dtype.float, Dims(i=2))
        assert list(g.keys()) == ["First", "Second"]
        lines = body(generate(g, namespace="demo"))
        assert lines[0] == "namespace demo {" and lines[-1] == "}  // namespace demo"
        assert lines.count("struct I_tag;") == 1   # shared dimension declared once


class TestErrors:
    def test_tensor_map_rules(self):
        with pytest.raises(ValueError, match="16 bytes"):
            TensorMapSpec(dtype.half, Dims(c=4, w=8))
        with pytest.raises(ValueError, match="swizzle span"):
            TensorMapSpec(dtype.half, Dims(c=128, w=8))          # 256 bytes > 128-byte swizzle
        with pytest.raises(ValueError, match="at most 256"):
            TensorMapSpec(dtype.half, Dims(c=64, w=512))
        with pytest.raises(ValueError, match="1 to 4 axes"):
            TensorMapSpec(dtype.half, Dims(c=64, w=2, h=2, n=2, t=2))

    def test_conflicting_names_and_missing_names(self):
        g = Generators()
        g.C8 = Fold("C", 8)
        g.X = Tensor(dtype.float, Dims(c4=2))
        g.C4 = Fold("C", 2)          # the tensor's implicit C4 is Fold<C, 4>
        with pytest.raises(ValueError, match="two different specifications"):
            generate(g)
        with pytest.raises(ValueError, match="has no name"):
            generate([Tensor(dtype.float, Dims(i=2))])

    def test_strides_must_not_overlap(self):
        with pytest.raises(ValueError, match="overlaps"):
            Tensor(dtype.float, Dims(i=4, k=8), Strides(i=4))
        with pytest.raises(ValueError, match="does not have"):
            Tensor(dtype.float, Dims(i=4), Strides(j=4))


def test_specs_embedded_in_a_source_file():
    src = """
    /*@spio
    I = Dim()
    I4 = Fold(I, 4)
    A = Tensor(dtype.float, Dims(I(16)))
    @spio*/
    int main() {}
    /*@spio
    Idx = CompoundIndex(Dims(I4(4), I(4)))
    @spio*/
    """
    g = extract_specs(src)
    assert list(g.keys()) == ["I", "I4", "A", "Idx"]
    assert body(generate_from_source(src))[-1] == (
        f"using Idx = {T}::CompoundIndex<{T}::Extent<I4, 4, 0>, {T}::Extent<I, 4, 0>>;")
    with pytest.raises(Exception):   # no builtins in the blocks' scope
        extract_specs("/*@spio\nX = open('/etc/passwd')\n@spio*/")


@pytest.mark.skipif(shutil.which("g++") is None, reason="needs a host C++ compiler")
def test_typed_header_lessons_compile_and_run_on_the_host(tmp_path):
    """tests/cpp/typed_lessons.cpp: type safety, position-free subscripting, folding, compound
    indices, with its types generated from its own @spio blocks."""
    src = ROOT / "tests" / "cpp" / "typed_lessons.cpp"
    (tmp_path / "types.h").write_text(generate_from_source(src.read_text()))
    exe = tmp_path / "lessons"
    subprocess.run(["g++", "-std=c++17", "-Wall", "-Werror", "-I", str(tmp_path), "-I", str(CSRC), str(src), "-o", str(exe)],
                   check=True, capture_output=True, text=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and "typed lessons ok" in out.stdout, out.stdout


def test_typed_kernel_compiles_for_sm_100a_and_misuse_does_not():
    src = (ROOT / "spio_b200" / "examples" / "typed_tile_copy.cu").read_text()
    header = {"types.h": generate_from_source(src)}
    cubin, log = compile_kernel(src, source_name="typed_tile_copy.cu", arch=(10, 0), header_dict=header,
                                return_log=True)
    assert len(cubin) > 1000 and "spill stores" in log and " 0 bytes spill stores" in log
    # the innermost TMA coordinate as a plain channel index: alignment cannot be guaranteed
    with pytest.raises(ValueError, match="multiple of 16 bytes"):
        compile_kernel(src.replace("n, h0, C8(0))", "n, h0, C(8))"), arch=(10, 0), header_dict=header)
    # an image index used on a tensor that has no image axis
    with pytest.raises(ValueError, match="no axis of this index's dimension"):
        compile_kernel(src.replace("*src[c8][w][h]", "*src[c8][w][n]"), arch=(10, 0), header_dict=header)


def test_fragments_params_and_macros():
    from spio_b200.generators import Fragment, FragmentType, Macro, ParamsSpec

    g = Generators()
    g.I, g.J, g.K = Dim(), Dim(), Dim()
    g.Acc = Fragment(FragmentType.M16_N8_F32_C, g.I, g.J)
    g.AFrag = Fragment(FragmentType.M16_K16_F16_A, g.I, "k")
    g.Block = ParamsSpec(dict(p=16, unroll=True, eps=1e-6))
    g.Names = Macro(dict(KERNEL_NAME="my_kernel"))
    text = generate(g)
    assert '#include "typed_mma.cuh"' in text
    lines = body(text)
    assert f"using Acc = {T}::MmaM16N8F32C<I, J>;" in lines
    assert f"using AFrag = {T}::MmaM16K16F16A<I, K>;" in lines
    assert "namespace Block {" in lines and "inline constexpr int p = 16;" in lines
    assert "inline constexpr bool unroll = true;" in lines and "inline constexpr float eps = 1e-06f;" in lines
    assert "#define KERNEL_NAME my_kernel" in text.splitlines()
    with pytest.raises(ValueError):
        ParamsSpec(dict(name="text"))
    with pytest.raises(ValueError):
        Fragment("M16_N8_F32_C", g.I, g.J)


def test_typed_mma_kernel_compiles_and_mismatched_fragments_do_not():
    src = (ROOT / "spio_b200" / "examples" / "typed_mma_tile.cu").read_text()
    header = {"types.h": generate_from_source(src)}
    cubin = compile_kernel(src, source_name="typed_mma_tile.cu", arch=(10, 0), header_dict=header)
    assert len(cubin) > 1000
    # a B operand whose columns are rows of C: the multiply-accumulate has no such overload
    wrong = src.replace("BFrag = Fragment(FragmentType.N8_K16_F16_B, J, K)", "BFrag = Fragment(FragmentType.N8_K16_F16_B, I, K)")
    with pytest.raises(ValueError):
        compile_kernel(wrong, arch=(10, 0), header_dict={"types.h": generate_from_source(wrong)})


def test_gw8_translation_unit_is_generated():
    unit = gw8_translation_unit("spio_conv2d_gw8_fprop__x", False, 3, 3, 2, 2, 2)
    assert unit.splitlines()[:3] == ['#include "conv2d_gw8_fwd.cuh"', "using namespace spio_b200;",
                                     "using Cfg = spio_b200::Gw8Config<3, 3, 2, 2, 2>;"]
    assert 'extern "C" __global__ void __launch_bounds__(Cfg::THREADS, 1)' in unit
    assert "conv2d_gw8_fwd_body<Cfg>(in_map, out_map, g, wgt, bias, ns, nob, status);" in unit
    # the just-in-time path compiles exactly this text; tpw counts 8-pixel tiles, the forward
    # kernel takes ceil(tpw / 2) 16-pixel blocks
    assert kernel_source("spio_conv2d_gw8_fprop__x", False, 3, 3, 2, 4, 2) == unit
    wunit = gw8_translation_unit("w", True, 5, 3, 1, 2, 1)
    assert "using Cfg = spio_b200::Gw8Config<5, 3, 1, 2, 1>;" in wunit
    assert wunit.count('extern "C" __global__') == 2 and "w__dbias(" in wunit
    with pytest.raises(ValueError):
        gw8_translation_unit("not a name", False, 3, 3, 2, 2, 2)


def test_gw8_kernel_specs_describe_the_operand_boxes():
    g = gw8_kernel_specs(3, 3, 2, 2, 2, box_w=64, nb=1, ring_slots=4)
    assert list(g.keys()) == ["Cfg", "StreamedMap", "TiledMap", "SlotRing"]
    assert g.StreamedMap.box_bytes == 64 * 64 * 4 * 2          # one ring slot: 32 KiB
    assert g.TiledMap.box.sizes == [64, 56, 2, 1]
    code = generate(g)
    assert f"using SlotRing = {T}::MbarrierRing<4>;" in code
    compile_kernel('#include "types.h"\nextern "C" __global__ void k() {}', arch=(10, 0), header_dict={"types.h": code})
