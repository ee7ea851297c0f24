"""Parity of the CUDA kernels, called through the C ABI, with the CPU oracle.

Mirrors the reference's kernel tests (tests/test_conv2d_gw8.py:110-201 via
spio/src_tests/run_test.py:26-125): outputs pre-filled with a dead value, every tile
configuration of a shape, tolerance from the accumulation depth -- plus the bound
max|err| <= 1e-2 * max|ref|.
"""

import pytest
import torch

from oracle import oracle as O
from spio_b200.cuda import get_device_attributes
from spio_b200.kernels import (Conv2dGw8Params, conv2d_gw8_kernel_factory,
                               conv2d_gw8_wgrad_kernel_factory)
from tests import capi
from tests.shapes import CFG1, CFG3, CFG4, REFERENCE_TEST_SHAPES, ident
from tests.test_oracle import load_golden

pytestmark = pytest.mark.gpu


def check_all(sh, has_bias, seed=11, tune=None, style="baseline", what=("fprop", "dgrad", "wgrad")):
    x, w, b, dy = O.make_inputs(sh, seed=seed, bias=has_bias, style=style)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    scale = 3.0 if style == "reference" else 1.0
    tag = f"{sh} bias={has_bias} tune={tune}"
    if "fprop" in what:
        O.assert_close(capi.fprop(xd, wd, bd, sh, tune), O.c_fprop(x, w, b, sh), sh, "fprop", tag, scale)
    if "dgrad" in what:
        O.assert_close(capi.dgrad(dyd, wd, sh, tune), O.c_dgrad(dy, w, sh), sh, "dgrad", tag, scale)
    if "wgrad" in what:
        O.assert_close(capi.wgrad(xd, dyd, sh, tune), O.c_wgrad(x, dy, sh), sh, "wgrad", tag)
    assert capi.status() == 0


@pytest.mark.parametrize("case", REFERENCE_TEST_SHAPES, ids=ident)
def test_reference_test_shapes(case):
    sh, has_bias = case
    check_all(sh, has_bias)


@pytest.mark.parametrize("case", REFERENCE_TEST_SHAPES[::7], ids=ident)
def test_reference_input_distribution(case):
    """randn clipped to +-3 with unscaled weights, as the reference's tests draw them."""
    sh, has_bias = case
    check_all(sh, has_bias, style="reference")


@pytest.mark.parametrize("idx", range(8))
def test_golden_vectors(idx):
    sh, t = load_golden()[idx]
    d = {k: capi.to_dev(v) for k, v in t.items()}
    O.assert_close(capi.fprop(d["x"], d["w"], d["bias"], sh), t["y"], sh, "fprop", f"golden {idx}", 3.0)
    O.assert_close(capi.dgrad(d["dy"], d["w"], sh), t["dx"], sh, "dgrad", f"golden {idx}", 3.0)
    O.assert_close(capi.wgrad(d["x"], d["dy"], sh), t["dw"], sh, "wgrad", f"golden {idx}")
    assert capi.status() == 0


def test_single_forward_configuration():
    check_all(CFG1, False, seed=1234)


@pytest.mark.parametrize("n", [1, 2, 4, 8, 16])
def test_batch_sweep_layer_small_batches(n):
    check_all(O.Shape(n, 64, 56, 56, 3, 3, 1, 1), False, seed=1235)


@pytest.mark.parametrize("c,hw", CFG3 + CFG4)
def test_channel_resolution_ladder_reduced_batch(c, hw):
    check_all(O.Shape(4 if hw > 14 else 16, c, hw, hw, 3, 3, 1, 1), c in (96, 192, 384), seed=1236)


@pytest.mark.parametrize("params", [
    Conv2dGw8Params(n=4, c=64, h=16, w=32, padding=1, r=3, s=3, has_bias=True),
    Conv2dGw8Params(n=3, c=72, h=28, w=28, padding=1, r=3, s=3),
    Conv2dGw8Params(n=2, c=64, h=12, w=40, padding=(2, 1), r=5, s=3),
    Conv2dGw8Params(n=6, c=72, h=7, w=7, padding=1, r=3, s=3, has_bias=True),
], ids=lambda p: p.encode())
def test_every_tile_configuration(params):
    """EVERY configuration of the kernel families' configuration spaces gives the oracle's
    result, as the reference's kernel tests run every configuration of a shape
    (tests/test_conv2d_gw8.py:110-201).  The oracle runs once per shape."""
    attr = get_device_attributes(0)
    sh = O.Shape(params.n, params.c, params.h, params.w, params.r, params.s, params.padding_h,
                 params.padding_w)
    x, w, b, dy = O.make_inputs(sh, seed=11, bias=params.has_bias)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    want_y, want_dx, want_dw = O.c_fprop(x, w, b, sh), O.c_dgrad(dy, w, sh), O.c_wgrad(x, dy, sh)
    counts = []
    configs = list(conv2d_gw8_kernel_factory.configs(params, attr))
    counts.append(len(configs))
    for cfg in configs:
        O.assert_close(capi.fprop(xd, wd, bd, sh, cfg.as_tune()), want_y, sh, "fprop", f"{sh} {cfg}")
    configs = list(conv2d_gw8_kernel_factory.configs(params, attr, igrad=True))
    counts.append(len(configs))
    for cfg in configs:
        O.assert_close(capi.dgrad(dyd, wd, sh, cfg.as_tune()), want_dx, sh, "dgrad", f"{sh} {cfg}")
    configs = list(conv2d_gw8_wgrad_kernel_factory.configs(params, attr))
    counts.append(len(configs))
    for cfg in configs:
        O.assert_close(capi.wgrad(xd, dyd, sh, cfg.as_tune()), want_dw, sh, "wgrad", f"{sh} {cfg}")
    assert min(counts) >= 20
    assert capi.status() == 0


@pytest.mark.parametrize("tune", [dict(grid=1), dict(grid=3), dict(grid=7, ns=2, nob=1),
                                  dict(grid=7, ns=3, nob=1, pps=1), dict(grid=1000), dict(ncb=1),
                                  dict(ncb=2, nb=2), dict(pps=1), dict(pps=2, grid=5)])
def test_small_grids_rings_and_tiles(tune):
    """Few CTAs (long spans crossing image and chunk boundaries), more CTAs than SMs, the
    smallest ring, narrow tiles."""
    check_all(O.Shape(5, 136, 14, 22, 3, 3, 1, 1), True, tune=tune)


def test_wgrad_is_deterministic_and_ignores_scratch_contents():
    sh = O.Shape(16, 64, 56, 56, 3, 3, 1, 1)
    x, w, b, dy = O.make_inputs(sh, seed=5, bias=False)
    xd, dyd = capi.to_dev(x), capi.to_dev(dy)
    a = capi.wgrad(xd, dyd, sh)
    b2 = capi.wgrad(xd, dyd, sh)
    assert torch.equal(a, b2)
    assert capi.status() == 0


def test_argument_errors_are_reported():
    from spio_b200 import _clib
    import ctypes

    lib = _clib.load()
    bad = _clib.Shape(1, 12, 8, 8, 3, 3, 1, 1)
    assert lib.spio_conv2d_gw8_fprop(1, 1, 1, None, ctypes.byref(bad), None, None) != 0
    assert "divisible by group width" in _clib.last_error()
    bad = _clib.Shape(1, 16, 8, 8, 6, 3, 1, 1)
    assert lib.spio_conv2d_gw8_dgrad(1, 1, 1, ctypes.byref(bad), None, None) != 0
    assert "between 1 and 5" in _clib.last_error()
    ok = _clib.Shape(1, 16, 8, 8, 3, 3, 1, 1)
    x = torch.zeros(64, device="cuda")
    assert lib.spio_conv2d_gw8_wgrad(x.data_ptr(), x.data_ptr(), x.data_ptr(), ctypes.byref(ok), None,
                                     x.data_ptr(), 16, None) != 0
    assert "scratch" in _clib.last_error()
    assert lib.spio_conv2d_gw8_fprop(x.data_ptr() + 2, x.data_ptr(), x.data_ptr(), None,
                                     ctypes.byref(ok), None, None) != 0
    assert "aligned" in _clib.last_error()
