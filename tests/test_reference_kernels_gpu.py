"""This package's kernels against the REFERENCE's own kernels, run on the same GPU on the same inputs.

``oracle/build_ref_kernels.py`` compiles the reference's ``spio/src/conv2d_gw8.cu`` and
``conv2d_gw8_wgrad.cu`` for sm_100a (from the reference checkout, where one is available) into
``oracle/_ref/``; here they are loaded with the driver-API module loader and launched as the
reference launches them.  Both sides compute fp16 x fp16 products with fp32 accumulation and round
once, in different summation orders, so results agree to the accumulation-depth tolerance the
reference's own tests use (spio/util/close.py:6-35); the CPU oracle arbitrates.  Skipped when the
cubins have not been built.
"""

import pytest
import torch

from oracle import oracle as O
from oracle import ref_kernels
from tests import capi

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not ref_kernels.available(), reason="oracle/_ref has not been built")]

SMALL = [(8, 64, 32, 32), (6, 72, 19, 23)]


@pytest.mark.parametrize("dims", SMALL, ids=str)
def test_against_the_reference_kernels(dims):
    n, c, h, w = dims
    sh = O.Shape(n, c, h, w, 3, 3, 1, 1)
    x, wt, _, dy = O.make_inputs(sh, seed=51, bias=False)
    xd, wd, dyd = (capi.to_dev(t) for t in (x, wt, dy))
    ours = {"fprop": capi.fprop(xd, wd, None, sh), "dgrad": capi.dgrad(dyd, wd, sh), "wgrad": capi.wgrad(xd, dyd, sh)}
    want = {"fprop": O.c_fprop(x, wt, None, sh), "dgrad": O.c_dgrad(dy, wt, sh), "wgrad": O.c_wgrad(x, dy, sh)}
    ran = 0
    for kind in ("fprop", "dgrad", "wgrad"):
        kernels = ref_kernels.kernels_for(kind, n, c, h, w)
        assert kernels, f"no reference {kind} kernel was built for {dims}"
        for k in kernels:
            k.load()
            if kind == "fprop":
                out = torch.full_like(xd, capi.DEAD_VALUE)
                k(out, xd, wd, None)
            elif kind == "dgrad":
                out = torch.full_like(xd, capi.DEAD_VALUE)
                k(out, dyd, wd)
            else:
                out = torch.zeros(c, 8, 3, 3, dtype=torch.float32, device="cuda:0").contiguous(memory_format=capi.CL)
                k(out, xd, dyd)
            torch.cuda.synchronize()
            # the reference's kernel is right (CPU oracle) ...
            O.assert_close(out, want[kind], sh, kind, f"reference kernel {k}")
            # ... and this package's kernel agrees with it
            O.assert_close(ours[kind], out.cpu(), sh, kind, f"ours vs reference kernel {k}")
            k.unload()
            ran += 1
    assert ran >= 6
    assert capi.status() == 0


def test_reference_kernels_refuse_other_shapes():
    k = ref_kernels.kernels_for("fprop", 8, 64, 32, 32)[0]
    x = torch.zeros(4, 64, 32, 32, dtype=torch.float16, device="cuda:0").contiguous(memory_format=capi.CL)
    w = torch.zeros(64, 8, 3, 3, dtype=torch.float16, device="cuda:0").contiguous(memory_format=capi.CL)
    with pytest.raises(ValueError, match="takes"):
        k.check([x, x, w])
