"""The ``spio::layernorm_2d`` PyTorch operator: LayerNorm over the channels of an NCHW tensor
in channels_last memory format (fp16 data, fp32 statistics, fp32 weight and bias).

The reference ships a forward kernel for this op (spio/src/layernorm_2d.cu) without an
operator around it; here forward and backward are wired to autograd and CUDA autocast.  The
device work is done by libspio_b200 on torch's current stream; CPU tensors raise.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _clib
from ..util.tensor_format import to_channels_last


def _check(x: torch.Tensor, weight, bias) -> Tuple[int, int]:
    if x.device.type != "cuda":
        raise ValueError("spio layernorm_2d runs on CUDA devices only (no CPU implementation)")
    assert x.dim() == 4, "expected an NCHW tensor"
    assert x.dtype == torch.float16
    assert weight is None or (weight.dtype == torch.float32 and weight.numel() == x.shape[1])
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == x.shape[1])
    n, c, h, w = x.shape
    return n * h * w, c


def _ptr(t: Optional[torch.Tensor]):
    return t.data_ptr() if t is not None else None


@torch.library.custom_op("spio::layernorm_2d", mutates_args=())
def layernorm_2d_op(x: torch.Tensor, weight: Optional[torch.Tensor], bias: Optional[torch.Tensor],
                    eps: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """(y fp16 channels_last, stats fp32 [n*h*w, 2] = mean and reciprocal standard deviation)."""
    rows, c = _check(x, weight, bias)
    x = to_channels_last(x)
    y = torch.empty_like(x)
    stats = torch.empty((rows, 2), device=x.device, dtype=torch.float32)
    w = weight.contiguous() if weight is not None else None
    b = bias.contiguous() if bias is not None else None
    with torch.cuda.device(x.device):
        _clib.check(_clib.load().spio_layernorm_2d_fwd(
            y.data_ptr(), stats.data_ptr(), x.data_ptr(), _ptr(w), _ptr(b), rows, c, float(eps),
            torch.cuda.current_stream(x.device).cuda_stream), "layernorm_2d")
    return y, stats


@layernorm_2d_op.register_fake
def _layernorm_2d_fake(x, weight, bias, eps):
    n, c, h, w = x.shape
    return (x.new_empty(x.shape).to(memory_format=torch.channels_last),
            x.new_empty((n * h * w, 2), dtype=torch.float32))


@torch.library.custom_op("spio::layernorm_2d_backward", mutates_args=())
def layernorm_2d_backward_op(grad_output: torch.Tensor, x: torch.Tensor, stats: torch.Tensor,
                             weight: Optional[torch.Tensor], needs_weight_grad: bool,
                             needs_bias_grad: bool) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(grad_input fp16, grad_weight fp32, grad_bias fp32); a gradient that was not asked for
    comes back as an empty tensor."""
    rows, c = _check(x, weight, None)
    assert grad_output.dtype == torch.float16 and grad_output.shape == x.shape
    grad_output, x = to_channels_last(grad_output, x)
    lib = _clib.load()
    dx = torch.empty_like(x)
    dw = torch.empty(c if needs_weight_grad else 0, device=x.device, dtype=torch.float32)
    db = torch.empty(c if needs_bias_grad else 0, device=x.device, dtype=torch.float32)
    w = weight.contiguous() if weight is not None else None
    with torch.cuda.device(x.device):
        nbytes = lib.spio_layernorm_2d_bwd_scratch_bytes(rows, c)
        scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
        _clib.check(lib.spio_layernorm_2d_bwd(
            dx.data_ptr(), dw.data_ptr() if needs_weight_grad else None,
            db.data_ptr() if needs_bias_grad else None, grad_output.data_ptr(), x.data_ptr(),
            stats.data_ptr(), _ptr(w), rows, c, scratch.data_ptr(), nbytes,
            torch.cuda.current_stream(x.device).cuda_stream), "layernorm_2d backward")
    return dx, dw, db


@layernorm_2d_backward_op.register_fake
def _layernorm_2d_backward_fake(grad_output, x, stats, weight, needs_weight_grad, needs_bias_grad):
    c = x.shape[1]
    return (x.new_empty(x.shape).to(memory_format=torch.channels_last),
            x.new_empty(c if needs_weight_grad else 0, dtype=torch.float32),
            x.new_empty(c if needs_bias_grad else 0, dtype=torch.float32))


def _setup_context(ctx, inputs, output):
    x, weight, bias, _eps = inputs
    _y, stats = output
    ctx.save_for_backward(x, stats, weight)
    ctx.has_bias = bias is not None


def _backward(ctx, grad_y, _grad_stats):
    x, stats, weight = ctx.saved_tensors
    need = ctx.needs_input_grad
    want_w = bool(need[1]) and weight is not None
    want_b = bool(need[2]) and ctx.has_bias
    dx, dw, db = layernorm_2d_backward_op(grad_y.to(dtype=torch.float16), x, stats, weight, want_w, want_b)
    return (dx if need[0] else None), (dw if want_w else None), (db if want_b else None), None


layernorm_2d_op.register_autograd(_backward, setup_context=_setup_context)


def _layernorm_2d_autocast(ks, x, weight, bias, eps):
    """Under CUDA autocast: data in fp16, weight / bias / statistics in fp32; the result comes
    back in the input's dtype."""
    in_dtype = x.dtype
    autocast = torch._C.DispatchKeySet("AutocastCUDA")
    with torch._C._ExcludeDispatchKeyGuard(autocast):
        y, stats = torch.ops.spio.layernorm_2d.default.redispatch(
            ks - autocast, x.to(dtype=torch.float16),
            weight.to(dtype=torch.float32) if weight is not None else None,
            bias.to(dtype=torch.float32) if bias is not None else None, eps)
    return y.to(dtype=in_dtype), stats


_fragment = torch.library.Library("spio", "FRAGMENT")
_fragment.impl("layernorm_2d", _layernorm_2d_autocast, "AutocastCUDA", with_keyset=True)


def layernorm_2d(x: torch.Tensor, weight: Optional[torch.Tensor] = None, bias: Optional[torch.Tensor] = None,
                 eps: float = 1e-6) -> torch.Tensor:
    """LayerNorm over dim 1 of an NCHW tensor (channels_last fp16 on a CUDA device)."""
    return layernorm_2d_op(x, weight, bias, eps)[0]
