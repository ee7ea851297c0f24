"""Seeded random shapes through the three kernels (default launch plan, i.e. what the operator
uses for shapes nobody tuned), checked against torch's fp32 convolution and its autograd on the
same device.  Covers the corners the curated shapes may miss: one-pixel images, widths around the
tile sizes, channel counts that leave partial chunks, every filter size with every legal padding,
batches smaller and larger than the number of SMs."""

import random

import pytest
import torch

from oracle import oracle as O
from tests import capi

pytestmark = pytest.mark.gpu


def random_shapes(seed, count):
    rng = random.Random(seed)
    out = []
    while len(out) < count:
        r, s = rng.randint(1, 5), rng.randint(1, 5)
        pad_h, pad_w = rng.randint(0, r - 1), rng.randint(0, s - 1)
        h = rng.choice([1, 2, 3, 7, 8, 9, 14, 15, 17, 28, 31, 56, 57])
        w = rng.choice([1, 5, 7, 8, 9, 15, 16, 17, 24, 33, 47, 48, 49, 56, 63, 64, 65, 70, 113])
        if h + 2 * pad_h < r or w + 2 * pad_w < s:
            continue
        c = 8 * rng.choice([1, 2, 7, 8, 9, 16, 17, 24, 40])
        n = rng.choice([1, 2, 3, 5, 8, 13, 37])
        if n * c * h * w > 6_000_000:
            continue
        out.append(O.Shape(n, c, h, w, r, s, pad_h, pad_w))
    return out


def torch_reference(x, w, b, dy, sh):
    """fp32 convolution and gradients on the GPU (TF32 off)."""
    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        xf = x.float().requires_grad_(True)
        wf = w.float().requires_grad_(True)
        y = torch.nn.functional.conv2d(xf, wf, b, padding=(sh.pad_h, sh.pad_w), groups=sh.c // 8)
        dx, dw = torch.autograd.grad(y, (xf, wf), dy.float())
    finally:
        torch.backends.cudnn.allow_tf32 = old
    return y.detach(), dx, dw


@pytest.mark.parametrize("seed", range(6))
def test_random_shapes(seed):
    for sh in random_shapes(1000 + seed, 12):
        x, w, b, dy = O.make_inputs(sh, seed=seed, bias=True)
        xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
        y_ref, dx_ref, dw_ref = torch_reference(xd, wd, bd, dyd, sh)
        O.assert_close(capi.fprop(xd, wd, bd, sh), y_ref, sh, "fprop", f"fuzz {sh}", 2.0)
        O.assert_close(capi.dgrad(dyd, wd, sh), dx_ref, sh, "dgrad", f"fuzz {sh}", 2.0)
        O.assert_close(capi.wgrad(xd, dyd, sh), dw_ref, sh, "wgrad", f"fuzz {sh}", 2.0)
        if sh.r <= 3 and sh.s <= 3:   # the tcgen05 kernel too
            O.assert_close(capi.fprop(xd, wd, bd, sh, {"engine": 2}), y_ref, sh, "fprop", f"fuzz tc {sh}", 2.0)
            O.assert_close(capi.dgrad(dyd, wd, sh, {"engine": 2}), dx_ref, sh, "dgrad", f"fuzz tc {sh}", 2.0)
    assert capi.status() == 0
