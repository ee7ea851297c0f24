"""Images at most 8 pixels wide: the forward kernel pairs two images in one 16-pixel block tile.

A block tile is the M = 16 of one warp-level MMA.  For a 7 x 7 (or narrower) image a tile of
16 consecutive pixels would be half empty, so its two 8-pixel halves are pixels 0-7 of two
consecutive images of the ring slot (``ncb = 1`` with an even ``nb``); the reference folds
images into M for the same reason (spio/kernels/conv2d_gw8_kernel.py:92-94,
``block_q = 16 // block_n``).  Parity against the CPU oracle through the C ABI, and
bit-equality with the unpaired layout (``ncb = 2``), which computes every output element with
the same sequence of MMAs.
"""

import ctypes

import pytest
import torch

from oracle import oracle as O
from spio_b200 import _clib
from tests import capi

pytestmark = pytest.mark.gpu

SHAPES = [
    # n, c, h, w, r, s, pad_h, pad_w
    O.Shape(2, 64, 7, 7, 3, 3, 1, 1),
    O.Shape(3, 72, 7, 7, 3, 3, 1, 1),       # odd batch, partial channel chunk
    O.Shape(16, 768, 7, 7, 3, 3, 1, 1),     # the last rung of the channel / resolution ladder
    O.Shape(37, 136, 7, 7, 3, 3, 1, 1),     # image groups that do not divide the batch
    O.Shape(9, 64, 8, 8, 3, 3, 1, 1),       # exactly 8 pixels wide
    O.Shape(5, 64, 9, 6, 5, 5, 2, 2),
    O.Shape(6, 128, 6, 5, 3, 3, 1, 1),
    O.Shape(4, 64, 20, 4, 3, 1, 1, 0),
    O.Shape(8, 64, 5, 3, 1, 3, 0, 1),
    O.Shape(7, 64, 7, 10, 3, 3, 1, 0),      # fprop output 8 wide (paired), dgrad output 10 wide (not)
    O.Shape(6, 64, 7, 7, 3, 3, 0, 0),       # output 5 x 5
    O.Shape(4, 64, 4, 2, 3, 3, 2, 2),       # padding wider than the image
    O.Shape(2, 64, 1, 1, 1, 1, 0, 0),
    O.Shape(10, 64, 7, 7, 4, 2, 2, 1),      # even filter sizes
]


def plan(kind, sh, tune=None):
    info = _clib.PlanInfo()
    _clib.check(_clib.load().spio_conv2d_gw8_plan(kind, ctypes.byref(capi.cshape(sh)), _clib.tune_ref(tune),
                                                  ctypes.byref(info)))
    return info.as_dict()


@pytest.mark.parametrize("sh", SHAPES, ids=str)
def test_paired_layout_matches_the_oracle(sh):
    x, w, b, dy = O.make_inputs(sh, seed=21, bias=True)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    if sh.q <= 8:
        assert plan(_clib.FPROP, sh)["ncb"] == 1      # the planner pairs by itself
    if sh.w <= 8:
        assert plan(_clib.DGRAD, sh)["ncb"] == 1
    O.assert_close(capi.fprop(xd, wd, bd, sh), O.c_fprop(x, w, b, sh), sh, "fprop", f"paired {sh}")
    O.assert_close(capi.dgrad(dyd, wd, sh), O.c_dgrad(dy, w, sh), sh, "dgrad", f"paired {sh}")
    O.assert_close(capi.wgrad(xd, dyd, sh), O.c_wgrad(x, dy, sh), sh, "wgrad", f"paired {sh}")
    assert capi.status() == 0


@pytest.mark.parametrize("sh", [SHAPES[1], SHAPES[3], SHAPES[5]], ids=str)
@pytest.mark.parametrize("tune", [dict(ncb=1, nb=2), dict(ncb=1, nb=4, pps=1), dict(ncb=1, nb=8, pps=1),
                                  dict(ncb=1, nb=2, grid=3), dict(ncb=1, nb=4, wpg=1, tpw=8, pps=1),
                                  dict(ncb=1, ns=2, nob=1)])
def test_paired_layout_is_bit_identical_to_the_unpaired_one(sh, tune):
    if sh.r * sh.s > 9 and (tune.get("nb", 0) > 4 or "wpg" in tune):
        pytest.skip("large filters hold fewer tiles per warp and have fewer built-in variants")
    x, w, b, dy = O.make_inputs(sh, seed=22, bias=True)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    unpaired = dict(ncb=2)
    assert plan(_clib.FPROP, sh, unpaired)["ncb"] == 2
    assert torch.equal(capi.fprop(xd, wd, bd, sh, tune), capi.fprop(xd, wd, bd, sh, unpaired))
    assert torch.equal(capi.dgrad(dyd, wd, sh, tune), capi.dgrad(dyd, wd, sh, unpaired))
    assert capi.status() == 0


def test_planner_rejects_odd_image_counts_per_slot():
    lib = _clib.load()
    info = _clib.PlanInfo()
    sh = capi.cshape(O.Shape(8, 64, 7, 7, 3, 3, 1, 1))
    for tune in (dict(ncb=1, nb=3), dict(ncb=1, nb=64)):
        assert lib.spio_conv2d_gw8_plan(_clib.FPROP, ctypes.byref(sh), _clib.tune_ref(tune), ctypes.byref(info)) != 0
        assert "even nb" in _clib.last_error()
    # a single image cannot be paired
    one = capi.cshape(O.Shape(1, 64, 7, 7, 3, 3, 1, 1))
    _clib.check(lib.spio_conv2d_gw8_plan(_clib.FPROP, ctypes.byref(one), None, ctypes.byref(info)))
    assert info.ncb == 2 and info.nb == 1
