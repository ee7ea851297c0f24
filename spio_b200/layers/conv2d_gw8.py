"""``Conv2dGw8``: an ``nn.Conv2d`` whose forward runs the group-width-8 kernels.

Same class surface as the reference's layer (spio/layers/conv2d_gw8.py:12-140): ``make``,
``match``, ``match_args``, ``from_torch_module``, the ``Params`` attribute and an
``nn.Conv2d``-compatible state dict (it subclasses ``nn.Conv2d`` and shares the original
module's parameters).  Weights stay fp32 and autocast feeds the operator fp16 copies.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import nn

from ..functional import conv2d_gw8
from ..kernels import Conv2dGw8Params


def _pair(value) -> Tuple[int, int]:
    return (value, value) if isinstance(value, int) else tuple(value)


class Conv2dGw8(nn.Conv2d):
    Params = Conv2dGw8Params

    @staticmethod
    def match_args(in_channels, out_channels, kernel_size, stride=1, dilation=1, groups=1,
                   padding_mode="zeros", **_ignored) -> bool:
        """True when these ``nn.Conv2d`` arguments describe a layer the kernels support:
        as many outputs as inputs, 8 channels per group, filter extents 1..5, unit stride and
        dilation, zero padding."""
        r, s = _pair(kernel_size)
        return (in_channels == out_channels
                and groups > 0 and in_channels // groups == 8 and in_channels % groups == 0
                and 1 <= r <= 5 and 1 <= s <= 5
                and _pair(stride) == (1, 1) and _pair(dilation) == (1, 1)
                and padding_mode == "zeros")

    @staticmethod
    def match(module: nn.Module) -> bool:
        """True for a plain ``nn.Conv2d`` (not already converted) that :meth:`match_args` accepts."""
        if not isinstance(module, nn.Conv2d) or isinstance(module, Conv2dGw8):
            return False
        if isinstance(module.padding, str):
            return False
        return Conv2dGw8.match_args(module.in_channels, module.out_channels, module.kernel_size,
                                    module.stride, module.dilation, module.groups,
                                    padding_mode=module.padding_mode)

    @staticmethod
    def make(*args, **kwargs) -> Optional[nn.Module]:
        """A new layer for ``nn.Conv2d`` constructor arguments, or None if they do not match."""
        return Conv2dGw8(*args, **kwargs) if Conv2dGw8.match_args(*args, **kwargs) else None

    @staticmethod
    def from_torch_module(conv2d: nn.Conv2d) -> "Conv2dGw8":
        """A layer that shares ``conv2d``'s weight and bias parameters."""
        if not Conv2dGw8.match(conv2d):
            raise ValueError(f"Conv2d {conv2d} does not match Conv2dGw8")
        layer = Conv2dGw8(conv2d.in_channels, conv2d.out_channels, conv2d.kernel_size,
                          stride=conv2d.stride, padding=conv2d.padding, groups=conv2d.groups,
                          bias=conv2d.bias is not None, device="meta")
        layer.weight = conv2d.weight
        layer.bias = conv2d.bias
        layer.train(conv2d.training)
        return layer

    def forward(self, x: torch.Tensor) -> torch.Tensor:  # pylint: disable=arguments-renamed
        pad_y, pad_x = _pair(self.padding)
        return conv2d_gw8(x, self.weight, self.bias, stride=1, padding_y=pad_y, padding_x=pad_x,
                          groups=self.groups)
