"""Shape parameters of a group-width-8 convolution.

Same fields, derived quantities, textual encoding and validation rules as the reference's
``Conv2dGw8Params`` (spio/kernels/conv2d_gw8_params.py:10-209), so that code written
against the reference (tests, benchmarks, logged parameter sets) keeps working.
"""

from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Tuple, Union

GROUP_WIDTH = 8
_ENCODED = re.compile(r"(\d+)n_(\d+)c_(\d+)h_(\d+)w_(\d+)py_(\d+)px_(\d+)r_(\d+)s_(b|nb)$")


def _pair(value) -> Tuple[int, int]:
    if isinstance(value, (tuple, list)):
        return int(value[0]), int(value[1])
    return int(value), int(value)


@dataclass(frozen=True)
class Conv2dGw8Params:
    """n, c, h, w: input extents; padding: int or (pad_h, pad_w); r, s: filter extents.

    The output has as many channels as the input (k == c); every group is 8 channels wide
    on both sides; stride and dilation are 1.
    """

    n: int
    c: int
    h: int
    w: int
    padding: Union[int, Tuple[int, int]] = 1
    r: int = 3
    s: int = 3
    has_bias: bool = False
    group_width: int = GROUP_WIDTH
    stride: int = 1

    # ------------------------------------------------------------ derived quantities
    @property
    def padding_h(self) -> int:
        return _pair(self.padding)[0]

    @property
    def padding_w(self) -> int:
        return _pair(self.padding)[1]

    @property
    def transpose_padding_h(self) -> int:
        """Padding of the equivalent convolution that computes the input gradient."""
        return self.r - 1 - self.padding_h

    @property
    def transpose_padding_w(self) -> int:
        return self.s - 1 - self.padding_w

    @property
    def groups(self) -> int:
        return self.c // self.group_width

    @property
    def k(self) -> int:
        return self.c

    @property
    def p(self) -> int:
        return self.h + 2 * self.padding_h - self.r + 1

    @property
    def q(self) -> int:
        return self.w + 2 * self.padding_w - self.s + 1

    @property
    def kernel_size(self) -> Tuple[int, int]:
        return (self.r, self.s)

    @property
    def input_shape(self) -> Tuple[int, int, int, int]:
        return (self.n, self.c, self.h, self.w)

    @property
    def output_shape(self) -> Tuple[int, int, int, int]:
        return (self.n, self.k, self.p, self.q)

    @property
    def weight_shape(self) -> Tuple[int, int, int, int]:
        return (self.k, self.group_width, self.r, self.s)

    @property
    def bias_shape(self) -> Tuple[int]:
        return (self.k,)

    # ------------------------------------------------------------ text form
    def encode(self) -> str:
        """``{n}n_{c}c_{h}h_{w}w_{py}py_{px}px_{r}r_{s}s_{b|nb}``, the kernel-name suffix."""
        return (f"{self.n}n_{self.c}c_{self.h}h_{self.w}w_{self.padding_h}py_{self.padding_w}px_"
                f"{self.r}r_{self.s}s_{'b' if self.has_bias else 'nb'}")

    @classmethod
    def decode(cls, string: str) -> "Conv2dGw8Params":
        m = _ENCODED.match(string)
        if m is None:
            raise ValueError("Invalid string representation.")
        n, c, h, w, py, px, r, s = (int(v) for v in m.groups()[:8])
        return cls(n=n, c=c, h=h, w=w, padding=(py, px), r=r, s=s, has_bias=m.group(9) == "b")

    # ------------------------------------------------------------ construction
    @staticmethod
    def from_tensors(inputs, weight, bias, padding=1) -> "Conv2dGw8Params":
        """From the arguments of a ``torch.nn.functional.conv2d`` call (logical NCHW shapes)."""
        assert bias is None or (bias.dim() == 1 and bias.shape[0] == weight.shape[0])
        n, c, h, w = inputs.shape
        k, width, r, s = weight.shape
        assert width == GROUP_WIDTH, "Only group width of 8 is supported."
        assert k == c, "Number of output channels must match number of input channels."
        params = Conv2dGw8Params(n=n, c=c, h=h, w=w, padding=padding, r=r, s=s,
                                 has_bias=bias is not None)
        params.validate()
        return params

    @staticmethod
    def from_torch_module(module, inputs) -> "Conv2dGw8Params":
        n, c, h, w = inputs.shape
        k, _width, r, s = module.weight.shape
        assert k == c, f"Number of output channels must match number of input channels. {k} != {c}"
        return Conv2dGw8Params(n=n, c=c, h=h, w=w, padding=module.padding, r=r, s=s,
                               has_bias=module.bias is not None)

    # ------------------------------------------------------------ validation
    def validate(self) -> None:
        assert self.n > 0 and self.c > 0 and self.h > 0 and self.w > 0
        assert self.padding_h >= 0 and self.padding_w >= 0
        assert self.c % self.group_width == 0, "Number of channels must be divisible by group width."
        assert 1 <= self.r <= 5, "Kernel height must be between 1 and 5."
        assert 1 <= self.s <= 5, "Kernel width must be between 1 and 5."

    def is_valid(self) -> bool:
        try:
            self.validate()
        except AssertionError:
            return False
        return True
