"""Tolerance checks for fp16-in / fp32-accumulate results.

Same rule as the reference's test helper (spio/util/close.py:6-35): the absolute
tolerance grows with the accumulation depth of an output element, the relative tolerance
is twice the fp16 precision.
"""

from __future__ import annotations

import torch

FLOAT16_PRECISION = 5e-4
FLOAT32_PRECISION = 1.19e-7


def tolerance_for_depth(acc_depth: int, abs_mean: float = 1.6, atol_fudge: float = 3.5,
                        rtol_fudge: float = 2.0):
    """(atol, rtol) for sums of ``acc_depth`` products of operands of mean magnitude ``abs_mean``."""
    return acc_depth * abs_mean * abs_mean * FLOAT32_PRECISION * atol_fudge, FLOAT16_PRECISION * rtol_fudge


def assert_all_close(actual: torch.Tensor, expected: torch.Tensor, atol: float = 0, rtol: float = 0,
                     msg: str = None, max_errors: int = 128) -> None:
    """Raise AssertionError listing the first offending elements."""
    exp = expected.float()
    act = actual.float()
    err = (act - exp).abs()
    tol = atol + rtol * exp.abs()
    bad = err > tol
    if not bool(bad.any()):
        return
    where = torch.nonzero(bad)
    lines = [f"Tensors not close: atol={atol}, rtol={rtol}"]
    for idx in where[:max_errors].tolist():
        i = tuple(idx)
        lines.append(f"{list(i)} actual ={float(act[i]):>10.6f} expected ={float(exp[i]):>10.6f} "
                     f"|diff| = {float(err[i]):>10.6f} > abs_diff_tol = {float(tol[i]):>10.6f}")
    if where.shape[0] > max_errors:
        lines.append(f"... and {where.shape[0] - max_errors} more")
    if msg is not None:
        lines.append(str(msg))
    raise AssertionError("\n".join(lines))


def assert_all_close_with_acc_depth(actual, expected, msg: str = None, acc_depth: int = None,
                                    abs_mean: float = 1.6, atol_fudge: float = 3.5,
                                    rtol_fudge: float = 2.0) -> None:
    atol, rtol = tolerance_for_depth(acc_depth, abs_mean, atol_fudge, rtol_fudge)
    assert_all_close(actual, expected, atol=atol, rtol=rtol, msg=msg)
