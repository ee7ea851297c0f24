"""The reference's real-model layer shapes and the shipped tuning tables.

``test_model_shapes`` runs all 81 layer shapes the reference keeps for its tests and performance
models (spio/src_tests/Conv2dGw8Params.dat; the reference's tests sample them,
tests/test_conv2d_gw8.py:34-107) through the three kernels at a reduced batch, against the CPU
oracle.  ``test_tuning_table_entries`` runs, for every shape of the headline configurations, the
configuration the shipped tuning table holds -- what the PyTorch operator launches -- and the
planner's default, against the oracle.
"""

import json
from pathlib import Path

import pytest
import torch

from oracle import oracle as O
from spio_b200.cuda import get_device_attributes
from spio_b200.kernels import (Conv2dGw8Params, conv2d_gw8_kernel_factory, conv2d_gw8_wgrad_kernel_factory)
from spio_b200.kernels.kernel_cache import perf_model_cache
from spio_b200.kernels.performance_model_cache import MODEL_DIR
from tests import capi
from tests.shapes import CFG3, CFG4, ident, load_model_shapes

pytestmark = pytest.mark.gpu


def reduced(sh):
    """The shape with a batch the oracle handles in about a second."""
    per_image = sh.c * sh.h * sh.w * sh.r * sh.s
    n = max(2, min(sh.n, 8, 150_000_000 // max(per_image * 8, 1)))
    return O.Shape(n, sh.c, sh.h, sh.w, sh.r, sh.s, sh.pad_h, sh.pad_w)


@pytest.mark.parametrize("case", load_model_shapes(), ids=ident)
def test_model_shapes(case):
    full, has_bias = case
    sh = reduced(full)
    x, w, b, dy = O.make_inputs(sh, seed=41, bias=has_bias)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    O.assert_close(capi.fprop(xd, wd, bd, sh), O.c_fprop(x, w, b, sh), sh, "fprop", str(sh))
    O.assert_close(capi.dgrad(dyd, wd, sh), O.c_dgrad(dy, w, sh), sh, "dgrad", str(sh))
    O.assert_close(capi.wgrad(xd, dyd, sh), O.c_wgrad(x, dy, sh), sh, "wgrad", str(sh))
    assert capi.status() == 0


def headline_params():
    out = [Conv2dGw8Params(n=8, c=64, h=32, w=32, padding=1, r=3, s=3)]
    out += [Conv2dGw8Params(n=n, c=64, h=56, w=56, padding=1, r=3, s=3) for n in (128, 256, 512, 2048)]
    out += [Conv2dGw8Params(n=256, c=c, h=hw, w=hw, padding=1, r=3, s=3) for c, hw in CFG3]
    out += [Conv2dGw8Params(n=256, c=c, h=hw, w=hw, padding=1, r=3, s=3, has_bias=True) for c, hw in CFG4]
    return out


@pytest.mark.parametrize("params", headline_params(), ids=lambda p: p.encode())
def test_tuning_table_entries(params):
    """The table entry of the full-size shape (the configuration depends on the batch only through
    images per slot, which the reduced batch still covers) and the planner's default."""
    attr = get_device_attributes(0)
    n = min(params.n, 8 if params.h > 14 else 24)
    sh = O.Shape(n, params.c, params.h, params.w, params.r, params.s, params.padding_h, params.padding_w)
    x, w, b, dy = O.make_inputs(sh, seed=43, bias=params.has_bias)
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    want = {"fprop": O.c_fprop(x, w, b, sh), "dgrad": O.c_dgrad(dy, w, sh), "wgrad": O.c_wgrad(x, dy, sh)}
    found = 0
    for name, factory, kw in (("fprop", conv2d_gw8_kernel_factory, {}),
                              ("dgrad", conv2d_gw8_kernel_factory, {"igrad": True}),
                              ("wgrad", conv2d_gw8_wgrad_kernel_factory, {})):
        cfg = perf_model_cache.predict_best_kernel(factory, params, torch.device("cuda:0"), **kw)
        table = json.loads((MODEL_DIR / f"tuned__{factory.get_kernel_name(**kw)}__sm_100a.json").read_text())
        found += params.encode() in table
        for tune in (cfg.as_tune(), None):
            tune = dict(tune, nb=min(tune.get("nb", 0), n)) if tune else None
            got = {"fprop": lambda: capi.fprop(xd, wd, bd, sh, tune), "dgrad": lambda: capi.dgrad(dyd, wd, sh, tune),
                   "wgrad": lambda: capi.wgrad(xd, dyd, sh, tune)}[name]()
            O.assert_close(got, want[name], sh, name, f"{params.encode()} {tune}")
    assert found == 3, f"{params.encode()} is missing from a shipped tuning table"
    assert capi.status() == 0
