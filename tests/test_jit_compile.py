"""Just-in-time compilation on the CPU: NVRTC produces sm_100a cubins of the kernel templates.

Follows the reference's compiler tests (tests/test_compiler.py: compile a small kernel and
check that a cubin comes back; error text on bad source), which need no GPU either.
"""

import ctypes

import pytest

from spio_b200 import _clib
from spio_b200.compiler import compile_cuda, compile_kernel, compile_kernel_configs, nvrtc_version, sm_from_arch
from spio_b200.compiler.compile_kernel import kernel_source
from spio_b200.cuda import B200_ATTRIBUTES
from spio_b200.kernels import (Conv2dGw8Params, conv2d_gw8_kernel_factory,
                               conv2d_gw8_wgrad_kernel_factory)
from spio_b200.kernels.conv2d_gw8_kernel import Conv2dGw8Config, compiled_variants
from spio_b200.kernels.conv2d_gw8_wgrad_kernel import Conv2dGw8WgradConfig
from spio_b200.kernels.jit_kernel import JitKernel
from spio_b200.kernels.kernel import Kernel

ELF_MAGIC = b"\x7fELF"


def test_nvrtc_version():
    major, minor = nvrtc_version()
    assert (major, minor) >= (12, 8)  # first release that accepts sm_100a


def test_sm_from_arch():
    assert sm_from_arch((10, 0)) == "sm_100a"
    assert sm_from_arch((8, 0)) == "sm_80"
    assert sm_from_arch("sm_100a") == "sm_100a"
    assert sm_from_arch(None) is None


def test_compile_plain_kernel():
    src = 'extern "C" __global__ void add(const float* x, const float* y, float* z) {' \
          " z[threadIdx.x] = x[threadIdx.x] + y[threadIdx.x]; }"
    cubin = compile_cuda(src, arch=(10, 0), src_name="add.cu")
    assert cubin[:4] == ELF_MAGIC and len(cubin) > 500


def test_compile_with_memory_header_and_log():
    src = '#include "my_types.h"\nextern "C" __global__ void k(my_t* p) { p[0] = 1; }'
    cubin, log = compile_cuda(src, arch="sm_100a", header_dict={"my_types.h": "typedef int my_t;"},
                              ptxas_verbose=True, return_log=True)
    assert cubin[:4] == ELF_MAGIC
    assert "registers" in log and "sm_100a" in log


def test_compile_error_carries_the_log():
    with pytest.raises(ValueError, match="Compilation error log:.*undefined"):
        compile_cuda('extern "C" __global__ void k(int* p) { p[0] = undefined_name; }', arch=(10, 0))


def test_compile_kernel_rejects_old_arch():
    with pytest.raises(ValueError, match="sm_100a"):
        compile_kernel("", arch=(8, 0))


@pytest.mark.parametrize("wgrad", [False, True])
@pytest.mark.parametrize("rs,wpg,tpw,pps", [((3, 3), 1, 3, 1), ((3, 3), 3, 1, 2), ((5, 5), 1, 2, 1), ((1, 1), 1, 6, 2)])
def test_kernel_templates_compile_outside_the_built_in_variants(wgrad, rs, wpg, tpw, pps):
    assert (wpg, tpw, pps) not in compiled_variants(*rs)
    name = "spio_conv2d_gw8_test"
    cubin, log = compile_kernel(kernel_source(name, wgrad, rs[0], rs[1], wpg, tpw, pps), arch=(10, 0),
                                return_log=True)
    assert cubin[:4] == ELF_MAGIC
    assert f"Compiling entry function '{name}' for 'sm_100a'" in log


def test_kernel_source_checks_the_name():
    with pytest.raises(ValueError):
        kernel_source("bad name;", False, 3, 3, 2, 2, 1)


def test_factory_chooses_jit_for_unknown_variants(monkeypatch):
    p = Conv2dGw8Params(n=4, c=64, h=32, w=32, r=3, s=3, padding=1)
    built_in = conv2d_gw8_kernel_factory.make_kernel(p, Conv2dGw8Config(wpg=2, tpw=4, pps=1))
    assert type(built_in) is Kernel
    jit = conv2d_gw8_kernel_factory.make_kernel(p, Conv2dGw8Config(wpg=1, tpw=3, pps=1))
    assert isinstance(jit, JitKernel)
    forced = conv2d_gw8_kernel_factory.make_kernel(p, Conv2dGw8Config(wpg=2, tpw=4, pps=1), jit=True)
    assert isinstance(forced, JitKernel)
    from spio_b200.compiler import flags

    token = flags.jit.set(True)
    try:
        assert isinstance(conv2d_gw8_kernel_factory.make_kernel(p, None), JitKernel)
    finally:
        flags.jit.reset(token)


def test_jit_kernel_compile_plans_and_names():
    p = Conv2dGw8Params(n=8, c=128, h=28, w=28, r=3, s=3, padding=1, has_bias=True)
    k = conv2d_gw8_kernel_factory.make_kernel(p, Conv2dGw8Config(wpg=1, tpw=3, pps=1), igrad=True)
    k.compile(B200_ATTRIBUTES)
    assert k.cubin[:4] == ELF_MAGIC
    assert k.function_name == f"spio_conv2d_gw8_dgrad__{p.encode()}__wpg1_tpw3_pps1"
    assert k.function_name.encode() in k.cubin
    assert k.plan["threads"] == (8 * 1 + 4) * 32 and k.plan["wpg"] == 1 and k.plan["tpw"] == 3
    assert "registers" in k.compile_log
    lp = k.launch_params
    assert lp.grid >= 1 and lp.block == k.plan["threads"]


def test_jit_kernel_with_open_configuration_takes_the_planner_choice():
    p = Conv2dGw8Params(n=8, c=64, h=16, w=16, r=3, s=3, padding=1)
    k = conv2d_gw8_wgrad_kernel_factory.make_kernel(p, None, jit=True)
    k.compile(B200_ATTRIBUTES)
    assert (k.plan["wpg"], k.plan["tpw"], k.plan["pps"]) in compiled_variants(3, 3)
    assert k.plan["threads"] == (8 * k.plan["wpg"] + 1) * 32


def test_plan_jit_rejects_what_cannot_run():
    lib = _clib.load()
    sh = _clib.Shape(4, 64, 32, 32, 3, 3, 1, 1)
    info = _clib.PlanInfo()
    for tune in ({"wpg": 4, "tpw": 2, "pps": 1}, {"wpg": 2, "tpw": 0, "pps": 1}, {"wpg": 2, "tpw": 2, "pps": 5}):
        t = _clib.make_tune(tune)
        assert lib.spio_conv2d_gw8_plan_jit(_clib.FPROP, ctypes.byref(sh), ctypes.byref(t), 148, 232448,
                                            ctypes.byref(info)) != 0
        assert b"just-in-time" in lib.spio_b200_last_error()
    # a column tile wider than the warps can hold
    t = _clib.make_tune({"wpg": 1, "tpw": 1, "pps": 1, "ncb": 4})
    assert lib.spio_conv2d_gw8_plan_jit(_clib.WGRAD, ctypes.byref(sh), ctypes.byref(t), 148, 232448,
                                        ctypes.byref(info)) != 0


def test_compile_kernel_configs_in_parallel():
    p = Conv2dGw8Params(n=4, c=64, h=24, w=24, r=3, s=3, padding=1)
    cfgs = [Conv2dGw8WgradConfig(wpg=w, tpw=t, pps=1) for w, t in ((1, 3), (1, 5), (2, 3), (3, 1))]
    kernels = compile_kernel_configs(conv2d_gw8_wgrad_kernel_factory, p, cfgs, B200_ATTRIBUTES)
    assert len(kernels) == 4 and all(k.cubin[:4] == ELF_MAGIC for k in kernels)
    assert len({k.function_name for k in kernels}) == 4


def test_module_load_needs_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("checks the error path of a machine without a GPU")
    from spio_b200.cuda.driver import Module

    with pytest.raises(ValueError, match="CUDA error"):
        Module().load_data(b"\x7fELF")


def test_tcgen05_kernel_compiles_just_in_time():
    """The tcgen05 / tensor-memory forward kernel goes through NVRTC like the others."""
    p = Conv2dGw8Params(n=8, c=128, h=28, w=40, r=3, s=3, padding=1)
    k = conv2d_gw8_kernel_factory.make_kernel(p, Conv2dGw8Config(engine=2), jit=True, igrad=True)
    assert isinstance(k, JitKernel)
    k.compile(B200_ATTRIBUTES)
    assert k.cubin[:4] == ELF_MAGIC and k.function_name.endswith("__tcgen05")
    assert k.plan["engine"] == 2 and k.plan["threads"] == 640
    assert "tcgen05" in k.source and "Gw8TcConfig<3, 3>" in k.source
    built_in = conv2d_gw8_kernel_factory.make_kernel(p, Conv2dGw8Config(engine=2))
    assert type(built_in) is Kernel
    with pytest.raises(ValueError):
        kernel_source("k", True, 3, 3, 0, 0, 1, engine=2)
