"""Python face of the CPU oracle for the gw8 convolution path.  TEST INFRASTRUCTURE ONLY.

Only tests/, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline leg may import
this module; nothing under ``spio_b200/`` does.  It offers two independent checkers:

* ``c_fprop / c_dgrad / c_wgrad`` -- the plain-C restatement in
  ``conv2d_gw8_oracle.c`` (fp16 operands, fp32 sums, one rounding), built by
  ``oracle/Makefile`` into ``oracle/_build/liboracle_gw8.so``;
* ``torch_fprop / torch_grads`` -- ``torch.nn.functional.conv2d`` on fp32 copies of the
  fp16 tensors with TF32 off, and ``torch.autograd.grad`` of it: exactly what the
  reference's own tests compare its kernels with
  (spio/src_tests/run_test.py:43-50, 84-102, 253-307).

Tolerances are the reference's (spio/util/close.py:6-35) and the stricter-or-looser
"max abs error <= 1e-2 * max abs reference" bound; both are provided here.

The reference implements this path only as CUDA kernels that its Python generators
specialise per shape and compile with NVRTC, so there is no CPU build of the reference
itself to put in ``oracle/_ref``.
"""

from __future__ import annotations

import ctypes
import subprocess
from dataclasses import dataclass
from pathlib import Path
from typing import Optional, Tuple

import numpy as np
import torch

ORACLE_DIR = Path(__file__).resolve().parent
LIB_PATH = ORACLE_DIR / "_build" / "liboracle_gw8.so"

_lib = None


def build(force: bool = False) -> Path:
    """Compile the C oracle with the Makefile next to this file."""
    src = ORACLE_DIR / "conv2d_gw8_oracle.c"
    if force or not LIB_PATH.exists() or LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(ORACLE_DIR), "-B" if force else "-s"], check=True,
                       capture_output=True)
    return LIB_PATH


def load():
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        lib = ctypes.CDLL(str(LIB_PATH))
        i, vp = ctypes.c_int, ctypes.c_void_p
        lib.oracle_conv2d_gw8_fprop.argtypes = [vp, vp, vp, vp] + [i] * 8
        lib.oracle_conv2d_gw8_dgrad.argtypes = [vp, vp, vp] + [i] * 8
        lib.oracle_conv2d_gw8_wgrad.argtypes = [vp, vp, vp] + [i] * 8
        lib.oracle_num_threads.restype = i
        lib.oracle_set_num_threads.argtypes = [i]
        for f in (lib.oracle_conv2d_gw8_fprop, lib.oracle_conv2d_gw8_dgrad,
                  lib.oracle_conv2d_gw8_wgrad, lib.oracle_set_num_threads):
            f.restype = None
        _lib = lib
    return _lib


def num_threads() -> int:
    return load().oracle_num_threads()


def set_num_threads(n: int) -> None:
    load().oracle_set_num_threads(int(n))


@dataclass(frozen=True)
class Shape:
    """Problem shape; the fields of the reference's Conv2dGw8Params
    (spio/kernels/conv2d_gw8_params.py:10-44)."""

    n: int
    c: int
    h: int
    w: int
    r: int = 3
    s: int = 3
    pad_h: int = 1
    pad_w: int = 1

    @property
    def p(self) -> int:
        return self.h + 2 * self.pad_h - self.r + 1

    @property
    def q(self) -> int:
        return self.w + 2 * self.pad_w - self.s + 1

    @property
    def groups(self) -> int:
        return self.c // 8

    def ints(self):
        return (self.n, self.c, self.h, self.w, self.r, self.s, self.pad_h, self.pad_w)


# ---------------------------------------------------------------- layouts

def nhwc(t: torch.Tensor) -> torch.Tensor:
    """Logical (N,C,H,W) tensor -> contiguous array in NHWC order (weights (K,8,R,S) ->
    [K][R][S][8]), i.e. the bytes of its channels_last form."""
    return t.permute(0, 2, 3, 1).contiguous()


def from_nhwc(a: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`nhwc`: an NHWC array viewed as a logical (N,C,H,W) tensor."""
    return a.permute(0, 3, 1, 2)


def _ptr(t: torch.Tensor) -> int:
    assert t.is_contiguous() and t.device.type == "cpu"
    return t.data_ptr()


# ---------------------------------------------------------------- C restatement

def c_fprop(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], sh: Shape) -> torch.Tensor:
    """x (N,C,H,W) fp16, w (C,8,R,S) fp16, bias (C,) fp32 or None -> y (N,C,P,Q) fp16."""
    xa, wa = nhwc(x.cpu()), nhwc(w.cpu())
    ba = bias.cpu().float().contiguous() if bias is not None else None
    ya = torch.empty((sh.n, sh.p, sh.q, sh.c), dtype=torch.float16)
    load().oracle_conv2d_gw8_fprop(_ptr(ya), _ptr(xa), _ptr(wa), _ptr(ba) if ba is not None else None,
                                   *sh.ints())
    return from_nhwc(ya)


def c_dgrad(dy: torch.Tensor, w: torch.Tensor, sh: Shape) -> torch.Tensor:
    """dy (N,C,P,Q) fp16, w (C,8,R,S) fp16 -> dx (N,C,H,W) fp16."""
    da, wa = nhwc(dy.cpu()), nhwc(w.cpu())
    xa = torch.empty((sh.n, sh.h, sh.w, sh.c), dtype=torch.float16)
    load().oracle_conv2d_gw8_dgrad(_ptr(xa), _ptr(da), _ptr(wa), *sh.ints())
    return from_nhwc(xa)


def c_wgrad(x: torch.Tensor, dy: torch.Tensor, sh: Shape) -> torch.Tensor:
    """x (N,C,H,W) fp16, dy (N,C,P,Q) fp16 -> dw (C,8,R,S) fp32."""
    xa, da = nhwc(x.cpu()), nhwc(dy.cpu())
    wa = torch.empty((sh.c, sh.r, sh.s, 8), dtype=torch.float32)
    load().oracle_conv2d_gw8_wgrad(_ptr(wa), _ptr(xa), _ptr(da), *sh.ints())
    return from_nhwc(wa)


# ---------------------------------------------------------------- torch fp32 reference

class _no_tf32:
    """TF32 and cuDNN autotuning off, as the reference's tests set them
    (spio/src_tests/run_test.py:253-307)."""

    def __enter__(self):
        self.prev = (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32,
                     torch.backends.cudnn.benchmark)
        torch.backends.cudnn.allow_tf32 = False
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.benchmark = False

    def __exit__(self, *exc):
        (torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32,
         torch.backends.cudnn.benchmark) = self.prev


def torch_fprop(x, w, bias, sh: Shape) -> torch.Tensor:
    """fp32 result of torch.nn.functional.conv2d on fp32 copies of the operands."""
    with _no_tf32():
        return torch.nn.functional.conv2d(
            x.float(), w.float(), None if bias is None else bias.float(), stride=1,
            padding=(sh.pad_h, sh.pad_w), groups=sh.groups)


def torch_grads(x, w, dy, sh: Shape) -> Tuple[torch.Tensor, torch.Tensor]:
    """(dx, dw) in fp32 from torch.autograd.grad of the fp32 convolution."""
    with _no_tf32():
        xf = x.float().detach().requires_grad_(True)
        wf = w.float().detach().requires_grad_(True)
        y = torch.nn.functional.conv2d(xf, wf, None, stride=1, padding=(sh.pad_h, sh.pad_w),
                                       groups=sh.groups)
        dx, dw = torch.autograd.grad(y, (xf, wf), dy.float())
    return dx, dw


# ---------------------------------------------------------------- inputs and tolerances

def make_inputs(sh: Shape, seed: int, bias: bool = True, style: str = "baseline"):
    """Seeded synthetic operands (CPU tensors, logical NCHW shapes).

    style "baseline": activations and output gradients ~N(0,1), weights ~N(0,1/sqrt(8RS)).
    style "reference": every operand randn clipped to +-3, weights unscaled -- the
    distribution of the reference's tests (spio/reflection/arg_info.py:81-85).
    """
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(sh.n, sh.c, sh.h, sh.w, generator=g)
    w = torch.randn(sh.c, 8, sh.r, sh.s, generator=g)
    b = torch.randn(sh.c, generator=g) if bias else None
    dy = torch.randn(sh.n, sh.c, sh.p, sh.q, generator=g)
    if style == "reference":
        x, w, dy = x.clip(-3, 3), w.clip(-3, 3), dy.clip(-3, 3)
        b = b.clip(-3, 3) if b is not None else None
    else:
        w = w / (8 * sh.r * sh.s) ** 0.5
    return x.half(), w.half(), (b.float() if b is not None else None), dy.half()


def acc_depth(sh: Shape, what: str) -> int:
    """Accumulation depth of an output element (spio/kernels/conv2d_stats.py:71-84,111-118)."""
    return sh.n * sh.h * sh.w if what == "wgrad" else 8 * sh.r * sh.s


def reference_tolerance(sh: Shape, what: str) -> Tuple[float, float]:
    """(atol, rtol) of the reference's assert_all_close_with_acc_depth (spio/util/close.py:6-35)."""
    atol = acc_depth(sh, what) * 1.6 * 1.6 * 1.19e-7 * 3.5
    rtol = 5e-4 * 2.0
    return atol, rtol


def assert_close(actual: torch.Tensor, expected: torch.Tensor, sh: Shape, what: str, msg: str = "",
                 atol_scale: float = 1.0) -> None:
    """Both bounds at once: |a - e| <= atol + rtol*|e| element-wise (reference tolerance), and
    max|a - e| <= 1e-2 * max|e| (the headline bound)."""
    a, e = actual.detach().float().cpu(), expected.detach().float().cpu()
    assert a.shape == e.shape, f"{msg}: shape {tuple(a.shape)} != {tuple(e.shape)}"
    atol, rtol = reference_tolerance(sh, what)
    atol *= atol_scale
    diff = (a - e).abs()
    bad = diff > atol + rtol * e.abs()
    if bool(bad.any()):
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(
            f"{msg} {what}: {int(bad.sum())} of {bad.numel()} elements off; first {idx} actual "
            f"{a[tuple(idx)]:.6f} expected {e[tuple(idx)]:.6f} (atol {atol:.3g}, rtol {rtol:.3g})")
    emax = float(e.abs().max())
    assert float(diff.max()) <= 1e-2 * emax + 1e-30, (
        f"{msg} {what}: max abs err {float(diff.max()):.4g} > 1e-2 * max abs ref {emax:.4g}")
