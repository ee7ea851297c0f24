"""The C-ABI library loads without a GPU, exports every symbol include/spio_b200.h declares,
and its device-free planner produces launches that respect the hardware limits."""

import ctypes
import re
from pathlib import Path

import pytest

from spio_b200 import _clib
from tests.shapes import REFERENCE_TEST_SHAPES, ident

HEADER = Path(__file__).resolve().parent.parent / "include" / "spio_b200.h"
SMS, SMEM = 148, 232448


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(spio_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    lib = _clib.load()
    names = declared_functions()
    assert len(names) >= 14
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert set(names) == set(_clib.SIGNATURES), "ctypes binding out of step with the header"
    assert b"sm_100a" in lib.spio_b200_version()


def test_struct_layouts_match_the_header():
    assert ctypes.sizeof(_clib.Shape) == 8 * 4
    assert ctypes.sizeof(_clib.Tune) == 9 * 4
    assert ctypes.sizeof(_clib.PlanInfo) == 16 * 4 + 8  # 16 ints, size_t


def plan(kind, sh, tune=None):
    lib = _clib.load()
    info = _clib.PlanInfo()
    s = _clib.Shape(sh.n, sh.c, sh.h, sh.w, sh.r, sh.s, sh.pad_h, sh.pad_w)
    rc = lib.spio_conv2d_gw8_plan_for(kind, ctypes.byref(s), _clib.tune_ref(tune), SMS, SMEM,
                                      ctypes.byref(info))
    return rc, info.as_dict()


@pytest.mark.parametrize("case", REFERENCE_TEST_SHAPES, ids=ident)
@pytest.mark.parametrize("kind", [_clib.FPROP, _clib.DGRAD, _clib.WGRAD])
def test_planner_respects_limits(case, kind):
    sh, _ = case
    rc, p = plan(kind, sh)
    assert rc == 0, _clib.last_error()
    assert 1 <= p["grid"] <= SMS
    assert p["smem_bytes"] <= SMEM - 1024
    if kind == _clib.WGRAD:   # tiles of 8 pixels x 2 rows
        assert p["nb"] * p["ncb"] <= p["wpg"] * p["tpw"]
    else:                     # blocks of 16 pixels x 1 row, (tpw + 1) // 2 per warp
        blocks = p["wpg"] * ((p["tpw"] + 1) // 2)
        out_w8 = ((sh.w if kind == _clib.DGRAD else sh.q) + 7) // 8
        if p["ncb"] == 1:     # images at most 8 pixels wide: two images share a block
            assert out_w8 == 1 and sh.n >= 2
            assert p["nb"] % 2 == 0 and p["nb"] // 2 <= blocks
        else:
            assert p["ncb"] >= 2
            assert p["nb"] * ((p["ncb"] + 1) // 2) <= blocks
    assert p["ns"] >= 2 and p["pps"] in (1, 2)
    assert p["threads"] % 32 == 0 and p["threads"] <= 1024
    out_w = sh.w if kind == _clib.DGRAD else sh.q
    out_h = sh.h if kind == _clib.DGRAD else sh.p
    assert p["n_col_tiles"] * p["ncb"] * 8 >= out_w
    assert p["n_pairs"] * 2 >= out_h
    assert p["n_image_groups"] * p["nb"] >= sh.n
    assert p["n_chunks"] * 64 >= sh.c
    if kind == _clib.WGRAD:
        assert p["scratch_bytes"] in (p["n_chunks"] * p["n_split"] * k * (64 * sh.r * sh.s * 8 + 64) * 4 for k in (1, p["wpg"]))
        assert p["grid"] == (p["n_split"] * p["n_chunks"] if p["n_chunks"] <= SMS else SMS)
    else:
        assert p["scratch_bytes"] == 0


def test_planner_rejects_bad_requests():
    from oracle.oracle import Shape

    lib = _clib.load()
    rc, _ = plan(_clib.FPROP, Shape(1, 12, 8, 8))
    assert rc != 0 and "divisible by group width" in _clib.last_error()
    rc, _ = plan(_clib.FPROP, Shape(1, 16, 8, 8, 6, 3))
    assert rc != 0 and "between 1 and 5" in _clib.last_error()
    rc, _ = plan(_clib.FPROP, Shape(1, 16, 2, 2, 5, 5, 0, 0))
    assert rc != 0 and "positive" in _clib.last_error()
    rc, _ = plan(_clib.FPROP, Shape(1, 16, 8, 8), dict(wpg=7))
    assert rc != 0 and "variant" in _clib.last_error()
    rc, _ = plan(_clib.FPROP, Shape(1, 64, 56, 56), dict(ns=16, nob=4, pps=1))
    assert rc != 0 and "shared memory" in _clib.last_error()
    assert lib.spio_conv2d_gw8_plan_for(9, None, None, SMS, SMEM, None) != 0


def test_headline_plan():
    from oracle.oracle import Shape

    rc, p = plan(_clib.FPROP, Shape(2048, 64, 56, 56))
    assert rc == 0 and p["grid"] == 148 and p["ncb"] == 7 and p["nb"] == 1 and p["n_pairs"] == 28
    rc, p = plan(_clib.WGRAD, Shape(2048, 64, 56, 56))
    assert rc == 0 and p["n_split"] == 148 and p["grid"] == 148


def test_planner_engine_2():
    """The tcgen05 forward kernel: 640 threads, one image and one 64-pixel row pair per slot."""
    from oracle.oracle import Shape

    sh = Shape(256, 64, 56, 56, 3, 3, 1, 1)
    rc, p = plan(_clib.FPROP, sh, {"engine": 2})
    assert rc == 0 and p["engine"] == 2 and p["threads"] == 640
    assert (p["ncb"], p["nb"], p["pps"], p["n_col_tiles"]) == (7, 1, 1, 1)
    assert 3 <= p["ns"] <= 8 and p["nob"] == 2
    assert p["smem_bytes"] == 1024 + p["ns"] * 16384 + 8192 + 2 * 9 * 2048 + 2 * 2 * 56 * 128
    assert p["smem_bytes"] <= SMEM - 6144
    rc, p = plan(_clib.DGRAD, Shape(8, 128, 20, 130, 1, 3, 0, 1), {"engine": 2})
    assert rc == 0 and p["n_col_tiles"] == 3 and p["n_chunks"] == 2
    rc, p = plan(_clib.FPROP, sh, None)
    assert rc == 0 and p["engine"] == 1
    assert plan(_clib.WGRAD, sh, {"engine": 2})[0] != 0
    assert plan(_clib.FPROP, Shape(8, 64, 20, 20, 5, 5, 2, 2), {"engine": 2})[0] != 0
    assert plan(_clib.FPROP, sh, {"engine": 2, "ncb": 8})[0] != 0
    assert plan(_clib.FPROP, sh, {"engine": 3})[0] != 0


def test_planner_keeps_rings_inside_the_196_kib_configuration():
    """The planner's own ring depth stops at the shared-memory soft cap while 3 (forward) or
    2 (weight gradient) slots remain; an explicit depth is taken as given."""
    from oracle.oracle import Shape

    cap = 194 * 1024
    rc, p = plan(_clib.FPROP, Shape(256, 64, 56, 56, 3, 3, 1, 1))
    assert rc == 0 and p["ns"] == 4 and p["smem_bytes"] <= cap
    rc, p = plan(_clib.DGRAD, Shape(256, 64, 56, 56, 3, 3, 1, 1), {"ns": 5})
    assert rc == 0 and p["ns"] == 5 and p["smem_bytes"] > cap
    # two row pairs per slot would leave the weight-gradient ring two slots deep under the cap:
    # the planner then streams one row pair per slot, which fits five
    rc, p = plan(_clib.WGRAD, Shape(256, 256, 28, 28, 3, 3, 1, 1))
    assert rc == 0 and p["pps"] == 1 and p["ns"] == 5 and p["smem_bytes"] <= cap
    rc, p = plan(_clib.WGRAD, Shape(256, 256, 28, 28, 3, 3, 1, 1), {"pps": 2})
    assert rc == 0 and p["ns"] == 2 and p["smem_bytes"] <= cap
    rc, p = plan(_clib.WGRAD, Shape(256, 256, 28, 28, 3, 3, 1, 1), {"pps": 2, "ns": 3})
    assert rc == 0 and p["ns"] == 3 and p["smem_bytes"] > cap
    rc, p = plan(_clib.WGRAD, Shape(256, 64, 56, 56, 3, 3, 1, 1))
    assert rc == 0 and p["pps"] == 2 and p["ns"] == 3
    # three slots of the 14 x 14 forward plan do not fit under the cap: the floor wins
    rc, p = plan(_clib.FPROP, Shape(256, 512, 14, 14, 3, 3, 1, 1))
    assert rc == 0 and p["ns"] == 3 and p["smem_bytes"] > cap
