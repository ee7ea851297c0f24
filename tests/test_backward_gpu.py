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
    assert lib.spio_conv2d_gw8_backward(dx.data_ptr(), None, xd.data_ptr(), dyd.data_ptr(), wd.data_ptr(),
                                        ctypes.byref(s), None, None, None, 0, st, None) == 0
    assert torch.equal(dx, capi.dgrad(dyd, wd, sh))
    assert lib.spio_conv2d_gw8_backward(None, None, xd.data_ptr(), dyd.data_ptr(), wd.data_ptr(),
                                        ctypes.byref(s), None, None, None, 0, st, None) != 0
    assert b"neither" in lib.spio_b200_last_error()
    assert capi.status() == 0
