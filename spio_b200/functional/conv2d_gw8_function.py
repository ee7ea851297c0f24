"""The ``spio::conv2d_gw8`` PyTorch operator and its backward.

Drop-in for the reference's operator (spio/functional/conv2d_gw8_function.py:17-233):
same operator names, signatures, argument checks, fake (meta) implementations, autograd
formula and AutocastCUDA rule.  The device work is done by the sm_100a kernels of
libspio_b200 on torch's current stream; there is no CPU implementation, CPU tensors
raise.
"""

from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from ..kernels import Conv2dGw8Params, conv2d_gw8_kernel_factory, conv2d_gw8_wgrad_kernel_factory
from ..kernels.kernel import launch_backward
from ..util.tensor_format import to_channels_last


# dtype of the grad_weight the backward operator returns.  float32 is the reference's contract
# (spio/functional/conv2d_gw8_function.py:127); with float16 the reduce step of the weight-gradient
# kernel rounds its fp32 sums once and stores the weight's own type, which saves the cast kernel
# autograd launches to hand an fp16 parameter (or autocast's fp16 copy of it) its gradient.
_grad_weight_dtype = torch.float32

# SPIO_CHECK_STATUS=1: every backward pass synchronises and checks the kernels' status word
# (spio_b200.check_status); off by default because of the synchronisation.
_CHECK_STATUS = os.environ.get("SPIO_CHECK_STATUS", "0") == "1"


def set_grad_weight_dtype(dtype: torch.dtype) -> None:
    """``torch.float32`` (default, as in the reference) or ``torch.float16``."""
    global _grad_weight_dtype
    if dtype not in (torch.float32, torch.float16):
        raise ValueError("grad_weight dtype must be torch.float32 or torch.float16")
    _grad_weight_dtype = dtype


def get_grad_weight_dtype() -> torch.dtype:
    return _grad_weight_dtype


def _is_unit(value) -> bool:
    return value in (1, (1, 1), [1, 1])


def _absent(like: torch.Tensor, dtype) -> torch.Tensor:
    return like.new_empty((0,), dtype=dtype)


def _require_cuda(t: torch.Tensor) -> None:
    if t.device.type != "cuda":
        raise ValueError("spio conv2d_gw8 runs on CUDA devices only (no CPU implementation)")


@torch.library.custom_op("spio::conv2d_gw8", mutates_args=())
def conv2d_gw8(
    inputs: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    stride: int = 1,
    padding_y: int = 0,
    padding_x: int = 0,
    dilation: int = 1,
    groups: int = 1,
) -> torch.Tensor:
    """2-D convolution with group width 8: fp16 channels_last tensors, fp32 accumulation.

    inputs (N, C, H, W) fp16; weight (C, 8, R, S) fp16; bias (C,) fp32 or None; stride and
    dilation must be 1; groups must equal C // 8.  Returns (N, C, P, Q) fp16 channels_last.
    """
    assert inputs.dtype == torch.float16
    assert weight.dtype == torch.float16
    assert bias is None or bias.dtype == torch.float32
    assert _is_unit(stride)
    assert _is_unit(dilation)
    assert groups == inputs.shape[1] // 8
    params = Conv2dGw8Params.from_tensors(inputs, weight, bias, (padding_y, padding_x))
    _require_cuda(inputs)
    output = torch.empty(params.output_shape, device=inputs.device, dtype=torch.float16,
                         memory_format=torch.channels_last)
    x, w = to_channels_last(inputs, weight)
    kernel = conv2d_gw8_kernel_factory.get_kernel(params, inputs.device)
    kernel(output, x, w, bias.contiguous() if bias is not None else None)
    return output


@conv2d_gw8.register_fake
def _conv2d_gw8_fake(inputs, weight, bias=None, stride: int = 1, padding_y: int = 0,
                     padding_x: int = 0, dilation: int = 1, groups: int = 1):
    assert _is_unit(stride)
    assert _is_unit(dilation)
    assert groups == inputs.shape[1] // 8
    params = Conv2dGw8Params.from_tensors(inputs, weight, bias, (padding_y, padding_x))
    return inputs.new_empty(params.output_shape).to(memory_format=torch.channels_last)


@torch.library.custom_op("spio::conv2d_gw8_backward", mutates_args=())
def conv2d_gw8_backward_op(
    inputs: torch.Tensor,
    weight: torch.Tensor,
    bias: Optional[torch.Tensor],
    grad_output: torch.Tensor,
    padding_y: int,
    padding_x: int,
    needs_input_grad: bool,
    needs_weight_grad: bool,
    needs_bias_grad: bool,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """(grad_input fp16, grad_weight fp32, grad_bias fp32).  A gradient that was not asked
    for comes back as an empty (0-element) tensor, because an operator schema cannot return
    None; :func:`conv2d_gw8_backward` turns those into None for autograd."""
    assert grad_output.dtype == torch.float16
    assert inputs.dtype == torch.float16
    assert weight.dtype == torch.float16
    _require_cuda(inputs)
    grad_output, inputs, weight = to_channels_last(grad_output, inputs, weight)
    params = Conv2dGw8Params.from_tensors(inputs, weight, bias, padding=(padding_y, padding_x))

    grad_weight = _absent(inputs, torch.float32)
    wgrad_kernel = dgrad_kernel = None
    if needs_weight_grad:
        # The kernel overwrites grad_weight, so no zero fill is needed.
        grad_weight = torch.empty(params.weight_shape, device=inputs.device, dtype=_grad_weight_dtype,
                                  memory_format=torch.channels_last)
        wgrad_kernel = conv2d_gw8_wgrad_kernel_factory.get_kernel(params, inputs.device)
    grad_input = _absent(inputs, torch.float16)
    if needs_input_grad:
        grad_input = torch.empty_like(inputs)
        dgrad_kernel = conv2d_gw8_kernel_factory.get_kernel(params, inputs.device, igrad=True)

    # With an odd number of filter taps the weight-gradient kernel sums grad_output over
    # n, h, w in the unused half of its last MMA; otherwise torch does that reduction.
    grad_bias = _absent(inputs, torch.float32)
    fused_bias = needs_bias_grad and needs_weight_grad and (params.r * params.s) % 2 == 1
    if needs_bias_grad:
        grad_bias = (torch.empty(params.k, device=inputs.device, dtype=torch.float32) if fused_bias
                     else grad_output.sum(dim=(0, 2, 3), dtype=torch.float32))

    if needs_weight_grad:
        # one call: the input-gradient kernel starts on SMs as the weight-gradient kernels free them
        launch_backward(wgrad_kernel, dgrad_kernel, grad_input, grad_weight, inputs, grad_output, weight,
                        grad_bias if fused_bias else None)
    elif needs_input_grad:
        dgrad_kernel(grad_input, grad_output, weight, None)
    if _CHECK_STATUS:
        from .. import check_status

        check_status()
    return grad_input, grad_weight, grad_bias


@conv2d_gw8_backward_op.register_fake
def _conv2d_gw8_backward_fake(inputs, weight, bias, _grad_output, _padding_y, _padding_x,
                              needs_input_grad, needs_weight_grad, needs_bias_grad):
    grad_weight = (weight.new_empty(weight.shape, dtype=_grad_weight_dtype)
                   .to(memory_format=torch.channels_last) if needs_weight_grad
                   else _absent(inputs, torch.float32))
    grad_bias = (bias.new_empty(bias.shape, dtype=torch.float32) if needs_bias_grad
                 else _absent(inputs, torch.float32))
    grad_input = (inputs.new_empty(inputs.shape).to(memory_format=torch.channels_last)
                  if needs_input_grad else _absent(inputs, torch.float16))
    return grad_input, grad_weight, grad_bias


def conv2d_gw8_backward(ctx, grad_output):
    inputs, weight, bias = ctx.saved_tensors
    need = ctx.needs_input_grad
    want = (need[0], need[1], need[2] and bias is not None)
    grads = conv2d_gw8_backward_op(inputs, weight, bias, grad_output, ctx.padding_y, ctx.padding_x,
                                   *want)
    grad_input, grad_weight, grad_bias = (g if w else None for g, w in zip(grads, want))
    return grad_input, grad_weight, grad_bias, None, None, None, None, None


def conv2d_gw8_setup_context(ctx, inputs, output):
    x, weight, bias, _stride, padding_y, padding_x, *_ = inputs
    assert x.dtype == torch.float16
    assert weight.dtype == torch.float16
    assert output.dtype == torch.float16
    assert bias is None or bias.dtype == torch.float32
    ctx.save_for_backward(x, weight, bias)
    ctx.padding_y = padding_y
    ctx.padding_x = padding_x


conv2d_gw8.register_autograd(conv2d_gw8_backward, setup_context=conv2d_gw8_setup_context)


def conv2d_gw8_autocast(ks, inputs, weight, bias, *args, **kwargs):
    """Under CUDA autocast: run in fp16 (bias in fp32) and return the input's dtype."""
    in_dtype = inputs.dtype
    bias16 = bias.to(dtype=torch.float32) if bias is not None else None
    autocast = torch._C.DispatchKeySet("AutocastCUDA")
    with torch._C._ExcludeDispatchKeyGuard(autocast):
        out = torch.ops.spio.conv2d_gw8.default.redispatch(
            ks - autocast, inputs.to(dtype=torch.float16), weight.to(dtype=torch.float16), bias16,
            *args, **kwargs)
    return out.to(dtype=in_dtype)


_fragment = torch.library.Library("spio", "FRAGMENT")
_fragment.impl("conv2d_gw8", conv2d_gw8_autocast, "AutocastCUDA", with_keyset=True)
