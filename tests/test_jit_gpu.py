"""Kernels compiled just in time with NVRTC and launched through the driver API, on the GPU.

Parity with the CPU oracle for tile configurations that are not built into the library, and
bit-equality with the built-in kernel for one that is (same template, same launch plan).
"""

import pytest
import torch

from oracle import oracle as O
from spio_b200.compiler import compile_cuda
from spio_b200.cuda import get_device_attributes
from spio_b200.cuda.driver import Module
from spio_b200.kernels import (Conv2dGw8Params, conv2d_gw8_kernel_factory,
                               conv2d_gw8_wgrad_kernel_factory)
from spio_b200.kernels.conv2d_gw8_kernel import Conv2dGw8Config, compiled_variants
from spio_b200.kernels.conv2d_gw8_wgrad_kernel import Conv2dGw8WgradConfig
from spio_b200.kernels.jit_kernel import JitKernel
from tests import capi

pytestmark = pytest.mark.gpu

CL = torch.channels_last


def params_of(sh, has_bias=False):
    return Conv2dGw8Params(n=sh.n, c=sh.c, h=sh.h, w=sh.w, r=sh.r, s=sh.s,
                           padding=(sh.pad_h, sh.pad_w), has_bias=has_bias)


def run(factory, p, cfg, args, jit=None, **kw):
    attr = get_device_attributes(0)
    k = factory.make_kernel(p, cfg, attr, jit=jit, **kw)
    k.compile(attr)
    k.load(0)
    k(*args)
    return k


def dead(shape, dtype):
    return torch.full(shape, capi.DEAD_VALUE, dtype=dtype, device="cuda:0").contiguous(memory_format=CL)


JIT_CASES = [
    (O.Shape(5, 72, 19, 23, 3, 3, 1, 1), (1, 3, 1)),
    (O.Shape(3, 128, 30, 40, 3, 3, 1, 1), (3, 1, 2)),
    (O.Shape(4, 64, 17, 17, 5, 5, 2, 2), (1, 2, 1)),
    (O.Shape(6, 136, 12, 50, 1, 1, 0, 0), (1, 6, 2)),
]


@pytest.mark.parametrize("sh,variant", JIT_CASES, ids=lambda v: str(v))
def test_jit_kernels_match_the_oracle(sh, variant):
    wpg, tpw, pps = variant
    assert variant not in compiled_variants(sh.r, sh.s)
    x, w, b, dy = O.make_inputs(sh, seed=5, bias=True)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    p = params_of(sh, has_bias=True)
    fcfg = Conv2dGw8Config(wpg=wpg, tpw=tpw, pps=pps)

    y = dead((sh.n, sh.c, sh.p, sh.q), torch.float16)
    k = run(conv2d_gw8_kernel_factory, p, fcfg, (y, xd, wd, bd))
    assert isinstance(k, JitKernel)
    use = k.resource_usage
    assert 0 < use["num_regs"] <= 255 and use["local_size_bytes"] <= 512
    O.assert_close(y, O.c_fprop(x, w, b, sh), sh, "fprop", f"jit {variant}")

    dx = dead((sh.n, sh.c, sh.h, sh.w), torch.float16)
    run(conv2d_gw8_kernel_factory, p, fcfg, (dx, dyd, wd, None), igrad=True)
    O.assert_close(dx, O.c_dgrad(dy, w, sh), sh, "dgrad", f"jit {variant}")

    dw = dead((sh.c, 8, sh.r, sh.s), torch.float32)
    run(conv2d_gw8_wgrad_kernel_factory, p, Conv2dGw8WgradConfig(wpg=wpg, tpw=tpw, pps=pps), (dw, xd, dyd))
    O.assert_close(dw, O.c_wgrad(x, dy, sh), sh, "wgrad", f"jit {variant}")
    assert capi.status() == 0


def test_jit_of_a_built_in_variant_is_bit_identical():
    sh = O.Shape(16, 64, 56, 56, 3, 3, 1, 1)
    x, w, b, dy = O.make_inputs(sh, seed=9, bias=True)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    p = params_of(sh, has_bias=True)
    cfg = Conv2dGw8Config(wpg=2, tpw=4, pps=1)
    out = []
    for jit in (False, True):
        y = dead((sh.n, sh.c, sh.p, sh.q), torch.float16)
        run(conv2d_gw8_kernel_factory, p, cfg, (y, xd, wd, bd), jit=jit)
        dw = dead((sh.c, 8, sh.r, sh.s), torch.float32)
        run(conv2d_gw8_wgrad_kernel_factory, p, Conv2dGw8WgradConfig(wpg=2, tpw=4, pps=2), (dw, xd, dyd), jit=jit)
        out.append((y, dw))
    assert torch.equal(out[0][0], out[1][0])
    assert torch.equal(out[0][1], out[1][1])
    assert capi.status() == 0


def test_function_launch_marshals_tensors_scalars_and_none():
    src = r'''
    extern "C" __global__ void axpb(float* y, const float* x, const float* opt, float a, int n, int b) {
      int i = blockIdx.x * blockDim.x + threadIdx.x;
      if (i < n) y[i] = a * x[i] + b + (opt ? opt[i] : 0.f);
    }'''
    module = Module()
    module.load_data(compile_cuda(src, arch=get_device_attributes(0).compute_capability))
    fn = module.get_function("axpb")
    assert fn.get_attribute("num_regs") > 0
    x = torch.arange(1000, dtype=torch.float32, device="cuda:0")
    y = torch.zeros_like(x)
    fn.launch((8,), (128,), [y, x, None, 2.5, 1000, 3])
    assert torch.equal(y, 2.5 * x + 3)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        fn.launch(8, 128, [y, x, x, 1.0, 1000, 0])
    side.synchronize()
    assert torch.equal(y, 2 * x)
    with pytest.raises(ValueError, match="unsupported kernel argument"):
        fn.launch(8, 128, [y, x, None, "a", 1000, 3])
    with pytest.raises(ValueError):
        module.get_function("no_such_kernel")
    module.unload()


def test_functional_path_with_jit_flag():
    """SPIO_JIT / flags.jit routes the operator through NVRTC-compiled kernels."""
    from spio_b200.compiler import flags
    from spio_b200.functional import conv2d_gw8

    sh = O.Shape(4, 64, 20, 20, 3, 3, 1, 1)
    x, w, b, dy = O.make_inputs(sh, seed=3, bias=True)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    caches = [conv2d_gw8_kernel_factory.get_kernel_cache(), conv2d_gw8_kernel_factory.get_kernel_cache(igrad=True),
              conv2d_gw8_wgrad_kernel_factory.get_kernel_cache()]
    for c in caches:
        c.clear_cache()
    token = flags.jit.set(True)
    try:
        xd.requires_grad_(True), wd.requires_grad_(True)
        y = conv2d_gw8(xd, wd, bd, padding_y=1, padding_x=1, groups=sh.c // 8)
        y.backward(dyd)
        kinds = [type(k) for c in caches for k in c._cache.values()]
        assert kinds and all(k is JitKernel for k in kinds)
    finally:
        flags.jit.reset(token)
        for c in caches:
            c.clear_cache()
    O.assert_close(y.detach(), O.c_fprop(x, w, b, sh), sh, "fprop", "jit functional")
    O.assert_close(xd.grad, O.c_dgrad(dy, w, sh), sh, "dgrad", "jit functional")
    O.assert_close(wd.grad.float(), O.c_wgrad(x, dy, sh), sh, "wgrad", "jit functional", 2.0)


def test_jit_tcgen05_kernel_is_bit_identical_to_the_built_in_one():
    sh = O.Shape(6, 136, 30, 56, 3, 3, 1, 1)
    x, w, b, dy = O.make_inputs(sh, seed=13, bias=True)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    p = params_of(sh, has_bias=True)
    cfg = Conv2dGw8Config(engine=2)
    out = []
    for jit in (False, True):
        y = dead((sh.n, sh.c, sh.p, sh.q), torch.float16)
        k = run(conv2d_gw8_kernel_factory, p, cfg, (y, xd, wd, bd), jit=jit)
        assert isinstance(k, JitKernel) == jit
        dx = dead((sh.n, sh.c, sh.h, sh.w), torch.float16)
        run(conv2d_gw8_kernel_factory, p, cfg, (dx, dyd, wd, None), jit=jit, igrad=True)
        out.append((y, dx))
    assert torch.equal(out[0][0], out[1][0]) and torch.equal(out[0][1], out[1][1])
    O.assert_close(out[1][0], O.c_fprop(x, w, b, sh), sh, "fprop", "jit tcgen05")
    O.assert_close(out[1][1], O.c_dgrad(dy, w, sh), sh, "dgrad", "jit tcgen05")
    assert capi.status() == 0


def test_jit_kernels_join_the_backward_chain_with_the_fused_bias_gradient():
    """Just-in-time kernels go through the same combined backward call as the built-in ones
    (cuLaunchKernelEx with the programmatic-dependent-launch attribute), including the
    instantiation that sums dy for the bias gradient; a built-in variant compiled just in time
    gives the built-in kernel's bits."""
    from spio_b200.kernels.kernel import launch_backward

    sh = O.Shape(24, 72, 28, 28, 3, 3, 1, 1)
    x, w, b, dy = O.make_inputs(sh, seed=17, bias=True)
    xd, wd, dyd = (capi.to_dev(t) for t in (x, w, dy))
    p = params_of(sh, has_bias=True)
    attr = get_device_attributes(0)
    out = []
    for jit in (False, True):
        wk = conv2d_gw8_wgrad_kernel_factory.make_kernel(p, Conv2dGw8WgradConfig(wpg=2, tpw=4, pps=2), attr, jit=jit)
        dk = conv2d_gw8_kernel_factory.make_kernel(p, Conv2dGw8Config(wpg=2, tpw=4, pps=2), attr, jit=jit, igrad=True)
        for k in (wk, dk):
            k.compile(attr)
            k.load(0)
            assert isinstance(k, JitKernel) == jit
        dx = dead((sh.n, sh.c, sh.h, sh.w), torch.float16)
        dw = dead((sh.c, 8, sh.r, sh.s), torch.float32)
        db = torch.full((sh.c,), capi.DEAD_VALUE, dtype=torch.float32, device="cuda:0")
        for _ in range(3):  # back to back: each call's kernels overlap the tail of the previous call's
            launch_backward(wk, dk, dx, dw, xd, dyd, wd, db)
        out.append((dx, dw, db))
    for a, b2 in zip(out[0], out[1]):
        assert torch.equal(a, b2)
    O.assert_close(out[1][0], O.c_dgrad(dy, w, sh), sh, "dgrad", "jit chain")
    O.assert_close(out[1][1], O.c_wgrad(x, dy, sh), sh, "wgrad", "jit chain")
    torch.testing.assert_close(out[1][2].cpu(), dy.float().sum(dim=(0, 2, 3)), rtol=1e-3, atol=5e-2)
    # a mixed chain: just-in-time weight gradient of a configuration that is not built in,
    # built-in input gradient
    wk = conv2d_gw8_wgrad_kernel_factory.make_kernel(p, Conv2dGw8WgradConfig(wpg=1, tpw=3, pps=1), attr)
    wk.compile(attr)
    wk.load(0)
    assert isinstance(wk, JitKernel)
    dk = conv2d_gw8_kernel_factory.make_kernel(p, Conv2dGw8Config(), attr, igrad=True)
    dk.compile(attr)
    dk.load(0)
    dx2, dw2 = dead((sh.n, sh.c, sh.h, sh.w), torch.float16), dead((sh.c, 8, sh.r, sh.s), torch.float32)
    db2 = torch.full((sh.c,), capi.DEAD_VALUE, dtype=torch.float32, device="cuda:0")
    launch_backward(wk, dk, dx2, dw2, xd, dyd, wd, db2)
    O.assert_close(dw2, O.c_wgrad(x, dy, sh), sh, "wgrad", "mixed chain")
    torch.testing.assert_close(db2, out[0][2], rtol=1e-4, atol=1e-2)
    assert torch.equal(dx2, capi.dgrad(dyd, wd, sh))
    assert capi.status() == 0


def test_jit_forward_kernel_replayed_from_a_cuda_graph():
    """A just-in-time launch recorded into a CUDA graph splits its work statically (it owns no
    dynamic-tail counters) and gives the bits of the live launch, replay after replay, also with
    another stream running the same kernel live beside it."""
    sh = O.Shape(64, 64, 56, 56, 3, 3, 1, 1)   # enough pairs per CTA for the dynamic tail
    x, w, b, _ = O.make_inputs(sh, seed=19, bias=True)
    xd, wd, bd = (capi.to_dev(t) for t in (x, w, b))
    p = params_of(sh, has_bias=True)
    attr = get_device_attributes(0)
    k = conv2d_gw8_kernel_factory.make_kernel(p, Conv2dGw8Config(wpg=2, tpw=4, pps=2), attr, jit=True)
    k.compile(attr)
    k.load(0)
    live = dead((sh.n, sh.c, sh.p, sh.q), torch.float16)
    k(live, xd, wd, bd)
    torch.cuda.synchronize()
    assert torch.equal(live, capi.fprop(xd, wd, bd, sh, dict(wpg=2, tpw=4, pps=2)))
    rec = dead((sh.n, sh.c, sh.p, sh.q), torch.float16)
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        k(rec, xd, wd, bd)
    other = dead((sh.n, sh.c, sh.p, sh.q), torch.float16)
    for _ in range(3):
        rec.fill_(capi.DEAD_VALUE)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            graph.replay()
        k(other, xd, wd, bd)   # live, on the current stream, while the replay runs on its own
        torch.cuda.synchronize()
        assert torch.equal(rec, live) and torch.equal(other, live)
    assert capi.status() == 0
