"""The combined backward entry point: weight gradient, reduce and input gradient chained with
programmatic dependent launch must give exactly what the separate entry points give, also
when the operands are produced by kernels launched just before it."""

import pytest
import torch

from oracle import oracle as O
from tests import capi
from tests.shapes import REFERENCE_TEST_SHAPES, ident

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("case", REFERENCE_TEST_SHAPES[::5], ids=ident)
def test_backward_equals_separate_calls(case):
    sh, _ = case
    x, w, _, dy = O.make_inputs(sh, seed=21, bias=False)
    xd, wd, dyd = (capi.to_dev(t) for t in (x, w, dy))
    dx, dw = capi.backward(xd, dyd, wd, sh)
    assert torch.equal(dx, capi.dgrad(dyd, wd, sh))
    assert torch.equal(dw, capi.wgrad(xd, dyd, sh))
    O.assert_close(dx, O.c_dgrad(dy, w, sh), sh, "dgrad", f"backward {sh}")
    O.assert_close(dw, O.c_wgrad(x, dy, sh), sh, "wgrad", f"backward {sh}")
    assert capi.status() == 0


def test_backward_follows_its_producers_in_stream_order():
    """dy and x are rewritten by torch kernels right before every call, and the results are
    consumed by torch kernels right after it; a kernel that ran ahead of its producers or
    behind its consumers would show up as a mismatch."""
    sh = O.Shape(32, 64, 56, 56, 3, 3, 1, 1)
    x, w, _, dy = O.make_inputs(sh, seed=4, bias=False)
    xd, wd, dyd = (capi.to_dev(t) for t in (x, w, dy))
    ref_dx, ref_dw = capi.dgrad(dyd, wd, sh), capi.wgrad(xd, dyd, sh)
    torch.cuda.synchronize()
    xs, dys = torch.empty_like(xd), torch.empty_like(dyd)
    for it in range(25):
        scale = float(2 ** (it % 3))  # powers of two: every product and sum scales exactly
        xs.zero_(), dys.zero_()
        torch.mul(xd, scale, out=xs)      # producers, queued immediately before the call
        torch.mul(dyd, scale, out=dys)
        dx, dw = capi.backward(xs, dys, wd, sh)
        dx_sum, dw_copy = dx.float().sum(), dw.clone()  # consumers, queued immediately after
        assert torch.equal(dw_copy, ref_dw * (scale * scale)), f"dw, iteration {it}"
        # exact except where the unscaled reference was rounded as an fp16 subnormal
        torch.testing.assert_close(dx.float(), ref_dx.float() * scale, rtol=0, atol=2e-7 * scale,
                                   msg=f"dx, iteration {it}")
        assert torch.isfinite(dx_sum)
    assert capi.status() == 0


def test_backward_single_gradient_and_errors():
    from spio_b200 import _clib
    import ctypes

    sh = O.Shape(4, 64, 16, 16, 3, 3, 1, 1)
    x, w, _, dy = O.make_inputs(sh, seed=2, bias=False)
    xd, wd, dyd = (capi.to_dev(t) for t in (x, w, dy))
    lib = _clib.load()
    s = capi.cshape(sh)
    dx = torch.empty_like(xd)
    st = torch.cuda.current_stream().cuda_stream
    assert lib.spio_conv2d_gw8_backward(dx.data_ptr(), None, None, xd.data_ptr(), dyd.data_ptr(), wd.data_ptr(),
                                        ctypes.byref(s), None, None, None, 0, st, None) == 0
    assert torch.equal(dx, capi.dgrad(dyd, wd, sh))
    assert lib.spio_conv2d_gw8_backward(None, None, None, xd.data_ptr(), dyd.data_ptr(), wd.data_ptr(),
                                        ctypes.byref(s), None, None, None, 0, st, None) != 0
    assert b"neither" in lib.spio_b200_last_error()
    assert capi.status() == 0


ODD_TAP_CASES = [case for case in REFERENCE_TEST_SHAPES if (case[0].r * case[0].s) % 2 == 1][::4]


@pytest.mark.parametrize("case", ODD_TAP_CASES, ids=ident)
def test_fused_bias_gradient(case):
    """dbias from the spare half of the weight-gradient MMA equals the fp64 sum of dy over
    n, h, w (dy is fp16, the kernel adds in fp32)."""
    sh, _ = case
    x, w, _, dy = O.make_inputs(sh, seed=33, bias=False)
    xd, wd, dyd = (capi.to_dev(t) for t in (x, w, dy))
    dx, dw, db = capi.backward(xd, dyd, wd, sh, with_bias=True)
    ref = dy.double().sum(dim=(0, 2, 3))
    scale = float(dy.double().abs().sum(dim=(0, 2, 3)).max())
    assert float((db.double().cpu() - ref).abs().max()) <= 1e-5 * scale + 1e-6
    assert torch.equal(dw, capi.wgrad(xd, dyd, sh))   # the weight gradient is unchanged by it
    assert torch.equal(dx, capi.dgrad(dyd, wd, sh))
    assert capi.status() == 0


def test_fused_bias_gradient_full_size_and_channel_tail():
    for sh in (O.Shape(64, 64, 56, 56, 3, 3, 1, 1), O.Shape(9, 200, 14, 14, 3, 3, 1, 1),
               O.Shape(5, 72, 9, 31, 5, 5, 2, 2), O.Shape(7, 136, 12, 12, 1, 1, 0, 0)):
        x, w, _, dy = O.make_inputs(sh, seed=1, bias=False)
        xd, wd, dyd = (capi.to_dev(t) for t in (x, w, dy))
        _, _, db = capi.backward(xd, dyd, wd, sh, with_bias=True)
        ref = dy.double().sum(dim=(0, 2, 3))
        scale = float(dy.double().abs().sum(dim=(0, 2, 3)).max())
        assert float((db.double().cpu() - ref).abs().max()) <= 1e-5 * scale + 1e-6, str(sh)
    assert capi.status() == 0


def test_fused_bias_gradient_rejects_even_taps():
    sh = O.Shape(4, 64, 16, 16, 2, 2, 0, 0)
    x, w, _, dy = O.make_inputs(sh, seed=2, bias=False)
    xd, wd, dyd = (capi.to_dev(t) for t in (x, w, dy))
    with pytest.raises(ValueError, match="odd number of filter taps"):
        capi.backward(xd, dyd, wd, sh, with_bias=True)


def test_step_host_matches_the_device_entry_points():
    """The pipelined host-buffer step (uploads, kernels and downloads of 32 pieces of the batch
    overlapping) returns bit for bit what the device-pointer entry points compute."""
    import ctypes

    from spio_b200 import _clib

    lib = _clib.load()
    for sh, with_bias in ((O.Shape(37, 64, 56, 56, 3, 3, 1, 1), True), (O.Shape(5, 72, 9, 20, 3, 3, 1, 1), False),
                          (O.Shape(40, 128, 14, 14, 5, 5, 2, 2), True)):
        x, w, b, dy = O.make_inputs(sh, seed=12, bias=with_bias)
        xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
        hx = x.permute(0, 2, 3, 1).contiguous().pin_memory()
        hdy = dy.permute(0, 2, 3, 1).contiguous().pin_memory()
        hw = w.permute(0, 2, 3, 1).contiguous().pin_memory()
        hb = b.contiguous().pin_memory() if with_bias else None
        hy = torch.empty(sh.n, sh.p, sh.q, sh.c, dtype=torch.float16).pin_memory()
        hdx = torch.empty(sh.n, sh.h, sh.w, sh.c, dtype=torch.float16).pin_memory()
        hdw = torch.empty(sh.c, sh.r, sh.s, 8, dtype=torch.float32).pin_memory()
        hdb = torch.empty(sh.c, dtype=torch.float32).pin_memory()
        s = capi.cshape(sh)
        for _ in range(2):   # the second call reuses the staging buffers and events
            hy.fill_(-1), hdx.fill_(-1), hdw.fill_(-1)
            _clib.check(lib.spio_conv2d_gw8_step_host(
                hy.data_ptr(), hdx.data_ptr(), hdw.data_ptr(), hdb.data_ptr(), hx.data_ptr(), hdy.data_ptr(),
                hw.data_ptr(), hb.data_ptr() if with_bias else None, ctypes.byref(s)))
            assert torch.equal(hy, capi.fprop(xd, wd, bd, sh).permute(0, 2, 3, 1).cpu())
            assert torch.equal(hdx, capi.dgrad(dyd, wd, sh).permute(0, 2, 3, 1).cpu())
            assert torch.equal(hdw, capi.wgrad(xd, dyd, sh).permute(0, 2, 3, 1).cpu())
            ref_db = dy.double().sum(dim=(0, 2, 3))
            assert float((hdb.double() - ref_db).abs().max()) <= 1e-5 * float(dy.double().abs().sum(dim=(0, 2, 3)).max()) + 1e-6
    assert capi.status() == 0


def test_step_is_capturable_in_a_cuda_graph():
    """fprop + the combined backward call (programmatic dependent launches, event record)
    captured into a CUDA graph and replayed give the results of the eager calls."""
    import ctypes

    from spio_b200 import _clib

    lib = _clib.load()
    sh = O.Shape(24, 64, 56, 56, 3, 3, 1, 1)
    x, w, b, dy = O.make_inputs(sh, seed=6, bias=True)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    ref_y, ref_dx, ref_dw = capi.fprop(xd, wd, bd, sh), capi.dgrad(dyd, wd, sh), capi.wgrad(xd, dyd, sh)
    s = capi.cshape(sh)
    y, dx = torch.empty_like(ref_y), torch.empty_like(ref_dx)
    dw = torch.empty_like(ref_dw)
    db = torch.empty(sh.c, dtype=torch.float32, device="cuda")
    nbytes = lib.spio_conv2d_gw8_wgrad_scratch_bytes(ctypes.byref(s), None)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    torch.cuda.synchronize()
    with torch.cuda.graph(graph, stream=side):
        sp = side.cuda_stream
        _clib.check(lib.spio_conv2d_gw8_fprop(y.data_ptr(), xd.data_ptr(), wd.data_ptr(), bd.data_ptr(),
                                              ctypes.byref(s), None, sp))
        _clib.check(lib.spio_conv2d_gw8_backward(dx.data_ptr(), dw.data_ptr(), db.data_ptr(), xd.data_ptr(),
                                                 dyd.data_ptr(), wd.data_ptr(), ctypes.byref(s), None, None,
                                                 scratch.data_ptr(), nbytes, sp, None))
    for _ in range(3):
        y.fill_(-1), dx.fill_(-1), dw.fill_(-1)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, ref_y) and torch.equal(dx, ref_dx) and torch.equal(dw, ref_dw)
    assert capi.status() == 0


@pytest.mark.parametrize("sh", [O.Shape(16, 64, 56, 56, 3, 3, 1, 1), O.Shape(6, 136, 14, 14, 5, 5, 2, 2),
                                O.Shape(8, 768, 7, 7, 3, 3, 1, 1)], ids=str)
def test_weight_gradient_in_the_parameters_own_type(sh):
    """With ``dw_f16`` the reduce step stores the fp32 sums rounded once to fp16: exactly the
    fp32 result passed through one round-to-nearest, which is what autograd's cast kernel would
    have produced from the reference's fp32 grad_weight."""
    import ctypes

    from spio_b200 import _clib

    x, w, _, dy = O.make_inputs(sh, seed=23, bias=False)
    xd, wd, dyd = (capi.to_dev(t) for t in (x, w, dy))
    lib = _clib.load()
    s = capi.cshape(sh)
    nbytes = lib.spio_conv2d_gw8_wgrad_scratch_bytes(ctypes.byref(s), None)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda:0")
    dw16 = torch.full((sh.c, 8, sh.r, sh.s), capi.DEAD_VALUE, dtype=torch.float16, device="cuda:0")
    dw16 = dw16.contiguous(memory_format=capi.CL)
    db = torch.full((sh.c,), capi.DEAD_VALUE, dtype=torch.float32, device="cuda:0")
    odd = (sh.r * sh.s) % 2 == 1
    opts = _clib.BackwardOpts(1, None, None, None)
    _clib.check(lib.spio_conv2d_gw8_backward_ex(
        None, dw16.data_ptr(), db.data_ptr() if odd else None, xd.data_ptr(), dyd.data_ptr(), wd.data_ptr(),
        ctypes.byref(s), None, None, scratch.data_ptr(), nbytes, torch.cuda.current_stream().cuda_stream, None,
        ctypes.byref(opts)))
    dw32 = capi.wgrad(xd, dyd, sh)
    assert torch.equal(dw16, dw32.half())
    if odd:
        torch.testing.assert_close(db.cpu(), dy.float().sum(dim=(0, 2, 3)), rtol=1e-3, atol=5e-2)
    assert capi.status() == 0


def test_operator_returns_fp16_weight_gradient_when_asked():
    from spio_b200.functional import conv2d_gw8_backward_op, get_grad_weight_dtype, set_grad_weight_dtype

    sh = O.Shape(8, 64, 20, 20, 3, 3, 1, 1)
    x, w, b, dy = O.make_inputs(sh, seed=29, bias=True)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    assert get_grad_weight_dtype() == torch.float32
    _, dw32, db32 = conv2d_gw8_backward_op(xd, wd, bd, dyd, 1, 1, False, True, True)
    set_grad_weight_dtype(torch.float16)
    try:
        _, dw16, db16 = conv2d_gw8_backward_op(xd, wd, bd, dyd, 1, 1, False, True, True)
    finally:
        set_grad_weight_dtype(torch.float32)
    assert dw32.dtype == torch.float32 and dw16.dtype == torch.float16
    assert torch.equal(dw16, dw32.half()) and torch.equal(db16, db32)
    assert capi.status() == 0
