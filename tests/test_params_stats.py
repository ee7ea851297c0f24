"""Params and Stats against values produced by the reference's own classes
(tests/golden/gw8_params_stats.json) and against the closed forms of the reference's
tests/test_stats.py."""

import json
from pathlib import Path

import pytest

from spio_b200.kernels import Conv2dGw8Params, Conv2dStats

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "gw8_params_stats.json").read_text())


def _params(row):
    kw = dict(row["params"])
    if isinstance(kw["padding"], list):
        kw["padding"] = tuple(kw["padding"])
    return Conv2dGw8Params(**kw)


@pytest.mark.parametrize("row", GOLDEN, ids=[r["encode"] for r in GOLDEN])
def test_params_match_reference(row):
    p = _params(row)
    assert p.encode() == row["encode"]
    assert Conv2dGw8Params.decode(row["encode"]).encode() == row["encode"]
    assert p.groups == row["groups"] and (p.p, p.q) == (row["p"], row["q"])
    assert [p.transpose_padding_h, p.transpose_padding_w] == row["transpose_padding"]
    assert list(p.input_shape) == row["input_shape"]
    assert list(p.output_shape) == row["output_shape"]
    assert list(p.weight_shape) == row["weight_shape"]
    assert list(p.bias_shape) == row["bias_shape"]


@pytest.mark.parametrize("row", GOLDEN, ids=[r["encode"] for r in GOLDEN])
@pytest.mark.parametrize("out", ["output", "grad_input", "grad_weight", "grad_bias"])
def test_stats_match_reference(row, out):
    st = Conv2dStats(_params(row), output_names=out)
    exp = row[out]
    assert st.macs == exp["macs"]
    assert st.bytes_read == exp["bytes_read"]
    assert st.bytes_written == exp["bytes_written"]
    assert st.bytes == exp["bytes"]
    assert st.accumulation_depths == exp["accumulation_depths"]


def test_stats_closed_forms():
    p = Conv2dGw8Params(n=16, h=32, w=64, c=128, r=3, s=3)
    act = 16 * 32 * 64 * 128
    st = Conv2dStats(p, output_names="output")
    assert st.bytes_read == (act + 128 * 8 * 9) * 2 and st.bytes_written == act * 2
    assert st.macs == act * 72 and st.accumulation_depths == [72]
    st = Conv2dStats(p, output_names="grad_weight")
    assert st.bytes_read == 2 * act * 2 and st.bytes_written == 128 * 72 * 2
    assert st.accumulation_depths == [16 * 32 * 64]
    both = Conv2dStats(p, output_names=["grad_input", "grad_weight"])
    assert both.macs == 2 * act * 72


def test_headline_bytes_formula():
    """B = 4*N*C*H*W + 144*C for 3x3 / pad 1 without bias."""
    for n in (1, 128, 512):
        p = Conv2dGw8Params(n=n, c=64, h=56, w=56)
        for out in ("output", "grad_input", "grad_weight"):
            assert Conv2dStats(p, output_names=out).bytes == 802816 * n + 9216


def test_params_validation_and_decode_errors():
    assert not Conv2dGw8Params(n=1, c=12, h=4, w=4).is_valid()
    assert not Conv2dGw8Params(n=1, c=16, h=4, w=4, r=6).is_valid()
    assert not Conv2dGw8Params(n=1, c=16, h=4, w=4, s=0).is_valid()
    assert Conv2dGw8Params(n=1, c=16, h=4, w=4, padding=(2, 0), r=4, s=1).is_valid()
    with pytest.raises(ValueError):
        Conv2dGw8Params.decode("not a kernel name")
    with pytest.raises(AssertionError):
        Conv2dGw8Params(n=0, c=16, h=4, w=4).validate()


def test_params_from_tensors_and_module():
    import torch

    x = torch.empty(2, 32, 9, 7, dtype=torch.float16)
    w = torch.empty(32, 8, 3, 5, dtype=torch.float16)
    b = torch.empty(32)
    p = Conv2dGw8Params.from_tensors(x, w, b, (1, 2))
    assert (p.n, p.c, p.h, p.w, p.r, p.s, p.has_bias) == (2, 32, 9, 7, 3, 5, True)
    assert p.output_shape == (2, 32, 9, 7)
    with pytest.raises(AssertionError):
        Conv2dGw8Params.from_tensors(x, torch.empty(32, 4, 3, 3), None)
    with pytest.raises(AssertionError):
        Conv2dGw8Params.from_tensors(x, torch.empty(64, 8, 3, 3), None)
    m = torch.nn.Conv2d(32, 32, 3, padding=1, groups=4, bias=False)
    p = Conv2dGw8Params.from_torch_module(m, x)
    assert p.padding == (1, 1) and not p.has_bias
