"""The C oracle is pinned against the reference's own oracle function and the fixtures
generated from the reference's Python code (tests/golden/make_golden.py)."""

import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests.shapes import FILTER_SIZES, GROUPS, PADDING, SANITY, ident

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_golden():
    z = np.load(GOLDEN / "gw8_cases.npz")
    meta = json.loads(bytes(z["meta"]).decode())
    cases = []
    for i, m in enumerate(meta):
        t = {k: torch.from_numpy(z[f"c{i}_{k}"]) for k in ("x", "w", "dy", "y", "dx", "dw")}
        t["bias"] = torch.from_numpy(z[f"c{i}_bias"]) if m["has_bias"] else None
        sh = O.Shape(m["n"], m["c"], m["h"], m["w"], m["r"], m["s"], m["pad_h"], m["pad_w"])
        assert (sh.p, sh.q) == (m["p"], m["q"])
        cases.append((sh, t))
    return cases


@pytest.mark.parametrize("idx", range(8))
def test_c_oracle_matches_golden_vectors(idx):
    sh, t = load_golden()[idx]
    O.assert_close(O.c_fprop(t["x"], t["w"], t["bias"], sh), t["y"], sh, "fprop", f"golden {idx}",
                   atol_scale=3.0)
    O.assert_close(O.c_dgrad(t["dy"], t["w"], sh), t["dx"], sh, "dgrad", f"golden {idx}",
                   atol_scale=3.0)
    O.assert_close(O.c_wgrad(t["x"], t["dy"], sh), t["dw"], sh, "wgrad", f"golden {idx}")


@pytest.mark.parametrize("idx", range(8))
def test_torch_reference_reproduces_golden_vectors(idx):
    """The fp32 torch reference used at test time is the function that made the fixtures."""
    sh, t = load_golden()[idx]
    y = O.torch_fprop(t["x"], t["w"], t["bias"], sh)
    dx, dw = O.torch_grads(t["x"], t["w"], t["dy"], sh)
    assert torch.allclose(y, t["y"], rtol=1e-5, atol=1e-5)
    assert torch.allclose(dx, t["dx"], rtol=1e-5, atol=1e-5)
    assert torch.allclose(dw, t["dw"], rtol=1e-5, atol=1e-4)


SMALL = [c for c in SANITY[:4] + FILTER_SIZES[::3] + PADDING[1:2] + GROUPS[:3]]


@pytest.mark.parametrize("case", SMALL, ids=ident)
@pytest.mark.parametrize("style", ["baseline", "reference"])
def test_c_oracle_matches_torch(case, style):
    sh, has_bias = case
    x, w, b, dy = O.make_inputs(sh, seed=7, bias=has_bias, style=style)
    # the reference distribution has unscaled weights: sums are ~sqrt(depth) larger
    scale = 3.0 if style == "reference" else 1.0
    O.assert_close(O.c_fprop(x, w, b, sh), O.torch_fprop(x, w, b, sh), sh, "fprop", ident(case),
                   atol_scale=scale)
    dx, dw = O.torch_grads(x, w, dy, sh)
    O.assert_close(O.c_dgrad(dy, w, sh), dx, sh, "dgrad", ident(case), atol_scale=scale)
    O.assert_close(O.c_wgrad(x, dy, sh), dw, sh, "wgrad", ident(case))


def test_oracle_empty_taps_and_thread_count():
    """Padding larger than the filter: border outputs see no input at all."""
    sh = O.Shape(1, 8, 3, 3, 1, 1, 2, 2)
    x, w, b, _ = O.make_inputs(sh, seed=1, bias=True)
    y = O.c_fprop(x, w, b, sh)
    assert tuple(y.shape) == (1, 8, 7, 7)
    assert torch.equal(y[0, :, 0, 0].float(), b.half().float())
    O.set_num_threads(1)
    assert O.num_threads() == 1
    y1 = O.c_fprop(x, w, b, sh)
    O.set_num_threads(0)
    assert torch.equal(y, y1)
