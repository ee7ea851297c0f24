"""The reference-side binding that the integration guide shows, executed: ``B200Kernel`` (a ctypes wrapper with the
call protocol of the reference's ``spio.kernels.Kernel``) against the CPU oracle, and the ``spio``
import name in a model script written for the reference."""

import pytest
import torch

from oracle import oracle as O
from tests import capi

pytestmark = pytest.mark.gpu


def test_b200_kernel_binding_matches_the_oracle():
    from spio_b200.examples.reference_binding import B200Kernel
    from spio_b200.kernels import Conv2dGw8Params, get_full_kernel_name

    sh = O.Shape(6, 72, 19, 23, 3, 3, 1, 1)
    params = Conv2dGw8Params(n=sh.n, c=sh.c, h=sh.h, w=sh.w, padding=1, r=3, s=3, has_bias=True)
    x, w, b, dy = O.make_inputs(sh, seed=61, bias=True)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    kernels = {kind: B200Kernel(get_full_kernel_name(f"spio_conv2d_gw8_{kind}", params), params)
               for kind in ("fprop", "dgrad", "wgrad")}
    for k in kernels.values():
        k.compile()
        k.load()
    y = torch.full_like(xd, capi.DEAD_VALUE)
    kernels["fprop"](y, xd, wd, bd)
    dx = torch.full_like(xd, capi.DEAD_VALUE)
    kernels["dgrad"](dx, dyd, wd, None)
    dw = torch.full((sh.c, 8, 3, 3), capi.DEAD_VALUE, dtype=torch.float32, device="cuda:0").contiguous(memory_format=capi.CL)
    kernels["wgrad"](dw, xd, dyd)
    O.assert_close(y, O.c_fprop(x, w, b, sh), sh, "fprop", "binding")
    O.assert_close(dx, O.c_dgrad(dy, w, sh), sh, "dgrad", "binding")
    O.assert_close(dw, O.c_wgrad(x, dy, sh), sh, "wgrad", "binding")
    assert capi.status() == 0
    bad = B200Kernel("spio_conv2d_gw8_fprop__x", params)
    with pytest.raises(ValueError, match="aligned"):
        bad(torch.empty(64, dtype=torch.float16, device="cuda:0")[1:], xd, wd, None)   # misaligned: reported, not launched


def test_model_script_written_for_the_reference_runs_under_the_spio_name():
    """The reference's usage: ``spio.transform.transform(model)`` swaps nn.Conv2d(groups=C/8) for
    ``spio.layers.Conv2dGw8`` (spio/transform/_transform.py:16-55, spio/layers/conv2d_gw8.py:12-129)."""
    import spio
    import spio.transform
    from spio.functional import conv2d_gw8
    from spio.kernels import Conv2dGw8Params
    from spio.layers import Conv2dGw8

    assert spio.supported_arch == ["sm_100a"]
    torch.manual_seed(7)
    model = torch.nn.Sequential(torch.nn.Conv2d(64, 64, 3, padding=1, groups=8), torch.nn.ReLU(),
                                torch.nn.Conv2d(64, 64, 3, padding=1, groups=8)).cuda()
    model = model.to(memory_format=torch.channels_last)      # fp32 parameters, fp16 under autocast
    x = torch.randn(4, 64, 20, 20, device="cuda").contiguous(memory_format=torch.channels_last)
    with torch.autocast("cuda", dtype=torch.float16):
        want = model(x)
    fast = spio.transform.transform(model)
    assert sum(isinstance(m, Conv2dGw8) for m in fast.modules()) == 2
    with torch.autocast("cuda", dtype=torch.float16):
        got = fast(x)
    torch.testing.assert_close(got.float(), want.float(), rtol=2e-2, atol=2e-2)
    xh, wh = x.half(), model[0].weight.detach().half().contiguous(memory_format=torch.channels_last)
    p = Conv2dGw8Params.from_tensors(xh, wh, model[0].bias, padding=1)
    y = conv2d_gw8(xh, wh, model[0].bias.detach(), padding_y=1, padding_x=1, groups=p.groups)
    with torch.autocast("cuda", dtype=torch.float16):
        ref = model[0](x)
    torch.testing.assert_close(y.float(), ref.float(), rtol=2e-2, atol=2e-2)
    assert capi.status() == 0
