"""The weight-gradient entry point that allocates nothing (spio_conv2d_gw8_wgrad_static).

Callers that cannot allocate device memory where they need the gradient -- a plugin inside
another framework's fixed memory pool, a loop that must not block on the allocator -- get the
same result as the ordinary entry point, with the scratch taken from a buffer built into the
library.  The file name sorts last so that a failure here cannot hide any other test.
"""

import ctypes

import pytest
import torch

from oracle import oracle as O
from spio_b200 import _clib
from tests import capi

pytestmark = pytest.mark.gpu


def wgrad_static(x, dy, sh, tune=None):
    lib = _clib.load()
    dw = torch.full((sh.c, 8, sh.r, sh.s), capi.DEAD_VALUE, dtype=torch.float32, device=x.device)
    dw = dw.contiguous(memory_format=capi.CL)
    s = capi.cshape(sh)
    rc = lib.spio_conv2d_gw8_wgrad_static(dw.data_ptr(), x.data_ptr(), dy.data_ptr(), ctypes.byref(s),
                                          _clib.tune_ref(tune), torch.cuda.current_stream().cuda_stream)
    return rc, dw


def test_static_scratch_matches_ordinary_entry_point_twice_in_a_row():
    shapes = [O.Shape(32, 64, 56, 56, 3, 3, 1, 1), O.Shape(6, 136, 14, 22, 3, 3, 1, 1)]
    for i, sh in enumerate(shapes):
        x, _, _, dy = O.make_inputs(sh, seed=40 + i, bias=False)
        xd, dyd = capi.to_dev(x), capi.to_dev(dy)
        expected = capi.wgrad(xd, dyd, sh)           # caller-provided scratch
        for call in range(2):                        # the shared buffer keeps the last call's contents
            rc, got = wgrad_static(xd, dyd, sh)
            assert rc == 0, _clib.last_error()
            assert capi.status() == 0
            if call == 1:
                # the property the entry point exists for: once the device is set up, a call takes
                # no memory from the driver (cudaMalloc would lower the free bytes) nor from torch's
                # allocator
                out = torch.full_like(got, capi.DEAD_VALUE)       # allocated BEFORE the measured call
                s = capi.cshape(sh)
                torch.cuda.synchronize()
                free_before, reserved_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved()
                rc = _clib.load().spio_conv2d_gw8_wgrad_static(
                    out.data_ptr(), xd.data_ptr(), dyd.data_ptr(), ctypes.byref(s), None,
                    torch.cuda.current_stream().cuda_stream)
                torch.cuda.synchronize()
                assert rc == 0, _clib.last_error()
                assert torch.cuda.mem_get_info()[0] == free_before, "the call took device memory from the driver"
                assert torch.cuda.memory_reserved() == reserved_before, "the call took memory from torch's allocator"
                assert torch.equal(out, expected)
            # same kernels, same fixed summation order: the results are identical
            assert torch.equal(got, expected), f"shape {i}, call {call}"
        O.assert_close(expected, O.c_wgrad(x, dy, sh), sh, "wgrad", "static scratch")


def test_static_scratch_rejects_shapes_beyond_its_size():
    sh = O.Shape(64, 64, 56, 56, 5, 5, 2, 2)         # 5x5 over all SMs needs more scratch than the buffer holds
    x = torch.zeros(sh.n, sh.c, sh.h, sh.w, dtype=torch.float16, device="cuda").contiguous(memory_format=capi.CL)
    rc, _ = wgrad_static(x, x, sh)
    assert rc != 0
    assert "built-in" in _clib.last_error() and "scratch" in _clib.last_error()
    rc, dw = wgrad_static(x, x, sh, tune=dict(grid=32))   # fewer CTAs -> fewer partials -> it fits
    assert rc == 0, _clib.last_error()
    assert capi.status() == 0 and float(dw.abs().max()) == 0.0
