"""Calls into libspio_b200 through its C ABI with torch CUDA tensors (test helper)."""

import ctypes

import torch

from spio_b200 import _clib

DEAD_VALUE = -42.0  # outputs are pre-filled so that an unwritten element is caught
CL = torch.channels_last


def cshape(sh):
    return _clib.Shape(sh.n, sh.c, sh.h, sh.w, sh.r, sh.s, sh.pad_h, sh.pad_w)


def to_dev(t, dev="cuda:0"):
    if t is None:
        return None
    t = t.to(dev)
    return t.contiguous(memory_format=CL) if t.dim() == 4 else t.contiguous()


def fprop(x, w, bias, sh, tune=None):
    lib = _clib.load()
    y = torch.full((sh.n, sh.c, sh.p, sh.q), DEAD_VALUE, dtype=torch.float16, device=x.device)
    y = y.contiguous(memory_format=CL)
    s = cshape(sh)
    _clib.check(lib.spio_conv2d_gw8_fprop(
        y.data_ptr(), x.data_ptr(), w.data_ptr(), bias.data_ptr() if bias is not None else None,
        ctypes.byref(s), _clib.tune_ref(tune), torch.cuda.current_stream().cuda_stream))
    return y


def dgrad(dy, w, sh, tune=None):
    lib = _clib.load()
    dx = torch.full((sh.n, sh.c, sh.h, sh.w), DEAD_VALUE, dtype=torch.float16, device=dy.device)
    dx = dx.contiguous(memory_format=CL)
    s = cshape(sh)
    _clib.check(lib.spio_conv2d_gw8_dgrad(
        dx.data_ptr(), dy.data_ptr(), w.data_ptr(), ctypes.byref(s), _clib.tune_ref(tune),
        torch.cuda.current_stream().cuda_stream))
    return dx


def wgrad(x, dy, sh, tune=None, scratch=None):
    lib = _clib.load()
    dw = torch.full((sh.c, 8, sh.r, sh.s), DEAD_VALUE, dtype=torch.float32, device=x.device)
    dw = dw.contiguous(memory_format=CL)
    s = cshape(sh)
    t = _clib.make_tune(tune)
    tref = ctypes.byref(t) if t is not None else None
    nbytes = lib.spio_conv2d_gw8_wgrad_scratch_bytes(ctypes.byref(s), tref)
    assert nbytes > 0, _clib.last_error()
    if scratch is None:
        # garbage on purpose: the kernel must not depend on the scratch contents
        scratch = torch.full((nbytes // 4,), float("nan"), dtype=torch.float32, device=x.device)
    _clib.check(lib.spio_conv2d_gw8_wgrad(
        dw.data_ptr(), x.data_ptr(), dy.data_ptr(), ctypes.byref(s), tref, scratch.data_ptr(),
        nbytes, torch.cuda.current_stream().cuda_stream))
    return dw


def status():
    return _clib.device_status()


def backward(x, dy, w, sh, dgrad_tune=None, wgrad_tune=None, with_bias=False):
    """(dx, dw) or (dx, dw, dbias) through the combined entry point."""
    lib = _clib.load()
    dx = torch.full((sh.n, sh.c, sh.h, sh.w), DEAD_VALUE, dtype=torch.float16, device=x.device)
    dx = dx.contiguous(memory_format=CL)
    dw = torch.full((sh.c, 8, sh.r, sh.s), DEAD_VALUE, dtype=torch.float32, device=x.device)
    dw = dw.contiguous(memory_format=CL)
    s = cshape(sh)
    nbytes = lib.spio_conv2d_gw8_wgrad_scratch_bytes(ctypes.byref(s), _clib.tune_ref(wgrad_tune))
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    db = torch.full((sh.c,), DEAD_VALUE, dtype=torch.float32, device=x.device) if with_bias else None
    _clib.check(lib.spio_conv2d_gw8_backward(
        dx.data_ptr(), dw.data_ptr(), db.data_ptr() if with_bias else None, x.data_ptr(), dy.data_ptr(),
        w.data_ptr(), ctypes.byref(s), _clib.tune_ref(dgrad_tune), _clib.tune_ref(wgrad_tune),
        scratch.data_ptr(), nbytes, torch.cuda.current_stream().cuda_stream, None))
    return (dx, dw, db) if with_bias else (dx, dw)
