"""The tcgen05 forward kernel (engine 2: UMMA from the TMA ring, accumulators in tensor memory)
against the CPU oracle, through the C ABI: fprop and dgrad for every filter size it supports,
column tiles, partial channel chunks, chunk changes inside a CTA's span, the ring wrap, odd
heights, paddings from 0 to r - 1, and the golden vectors."""

import pytest
import torch

from oracle import oracle as O
from tests import capi
from tests.shapes import REFERENCE_TEST_SHAPES, ident
from tests.test_oracle import load_golden

pytestmark = pytest.mark.gpu

TC = {"engine": 2}


def eligible(sh):
    return sh.r <= 3 and sh.s <= 3


def check(sh, has_bias=True, seed=17, tune=TC, scale=1.0):
    x, w, b, dy = O.make_inputs(sh, seed=seed, bias=has_bias)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    O.assert_close(capi.fprop(xd, wd, bd, sh, tune), O.c_fprop(x, w, b, sh), sh, "fprop", f"tc {sh} {tune}", scale)
    O.assert_close(capi.dgrad(dyd, wd, sh, tune), O.c_dgrad(dy, w, sh), sh, "dgrad", f"tc {sh} {tune}", scale)
    assert capi.status() == 0


@pytest.mark.parametrize("case", [c for c in REFERENCE_TEST_SHAPES if eligible(c[0])], ids=ident)
def test_reference_test_shapes(case):
    sh, has_bias = case
    check(sh, has_bias)


@pytest.mark.parametrize("r,s", [(r, s) for r in (1, 2, 3) for s in (1, 2, 3)])
def test_every_filter_size_and_padding(r, s):
    for pad_h in range(r):
        for pad_w in range(s):
            check(O.Shape(3, 72, 13, 45, r, s, pad_h, pad_w), seed=r * 10 + s)


@pytest.mark.parametrize("sh", [
    O.Shape(2, 64, 56, 56, 3, 3, 1, 1),     # the headline layer
    O.Shape(2, 64, 17, 130, 3, 3, 1, 1),    # three column tiles
    O.Shape(2, 64, 9, 64, 1, 1, 0, 0),      # 64-pixel tiles (s = 1)
    O.Shape(6, 200, 11, 24, 3, 3, 1, 1),    # four chunks, the last one partial
    O.Shape(1, 64, 1, 8, 3, 3, 1, 1),       # a single row
    O.Shape(5, 768, 7, 7, 3, 3, 1, 1),      # many chunks per CTA span
], ids=str)
def test_shapes(sh):
    check(sh)


@pytest.mark.parametrize("tune", [{"engine": 2, "ns": 3}, {"engine": 2, "ns": 5, "nob": 3},
                                  {"engine": 2, "grid": 7}, {"engine": 2, "ncb": 3}, {"engine": 2, "nob": 4}], ids=str)
def test_ring_and_grid_settings(tune):
    check(O.Shape(9, 128, 30, 56, 3, 3, 1, 1), tune=tune)


@pytest.mark.parametrize("idx", range(8))
def test_golden_vectors(idx):
    sh, t = load_golden()[idx]
    if not eligible(sh):
        pytest.skip("filter larger than 3 x 3")
    d = {k: capi.to_dev(v) for k, v in t.items()}
    O.assert_close(capi.fprop(d["x"], d["w"], d["bias"], sh, TC), t["y"], sh, "fprop", f"golden {idx}", 3.0)
    O.assert_close(capi.dgrad(d["dy"], d["w"], sh, TC), t["dx"], sh, "dgrad", f"golden {idx}", 3.0)
    assert capi.status() == 0


def test_full_size_batch_slices_agree():
    """At the benchmark's size the kernel must give each image the result it gets alone."""
    sh = O.Shape(300, 64, 56, 56, 3, 3, 1, 1)
    x, w, b, _ = O.make_inputs(sh, seed=8, bias=True)
    xd, wd, bd = (capi.to_dev(t) for t in (x, w, b))
    y = capi.fprop(xd, wd, bd, sh, TC)
    for n0 in (0, 149, 299):
        one = O.Shape(1, 64, 56, 56, 3, 3, 1, 1)
        assert torch.equal(y[n0:n0 + 1], capi.fprop(xd[n0:n0 + 1].contiguous(memory_format=torch.channels_last), wd, bd, one, TC))
    assert capi.status() == 0


def test_rejections():
    from spio_b200 import _clib

    x, w, b, dy = O.make_inputs(O.Shape(2, 64, 16, 16, 5, 5, 2, 2), seed=1, bias=False)
    with pytest.raises(ValueError, match="3 x 3"):
        capi.fprop(capi.to_dev(x), capi.to_dev(w), None, O.Shape(2, 64, 16, 16, 5, 5, 2, 2), TC)
    sh = O.Shape(2, 64, 16, 16, 3, 3, 1, 1)
    x, w, b, dy = O.make_inputs(sh, seed=1, bias=False)
    with pytest.raises((ValueError, AssertionError), match="fprop and dgrad only"):
        capi.wgrad(capi.to_dev(x), capi.to_dev(dy), sh, TC)
    with pytest.raises(ValueError, match="64 pixels"):
        capi.fprop(capi.to_dev(x), capi.to_dev(w), None, sh, {"engine": 2, "ncb": 8})
    assert _clib.device_status() == 0
