"""Algorithmic MACs and bytes of the convolution's four outputs.

The roofline figures of this project are computed from these counts: every tensor
element, weights and weight gradients included, is charged ``unit`` (2) bytes, reads and
writes are ideal (each operand once), and a bias add counts as half a MAC.  Same formulas
as the reference's ``Conv2dStats`` (spio/kernels/conv2d_stats.py:8-126).
"""

from __future__ import annotations

from math import prod

from .stats import Stats


class Conv2dStats(Stats):
    # element counts
    @property
    def _x(self) -> int:
        return prod(self.params.input_shape)

    @property
    def _y(self) -> int:
        return prod(self.params.output_shape)

    @property
    def _w(self) -> int:
        return prod(self.params.weight_shape)

    @property
    def _b(self) -> int:
        return prod(self.params.bias_shape) if self.params.has_bias else 0

    @property
    def _depth(self) -> int:
        return self.params.r * self.params.s * self.params.group_width

    # output = conv(input, weight) + bias
    @property
    def output_macs(self):
        return self._y * self._depth + (self._y / 2 if self.params.has_bias else 0)

    @property
    def output_bytes_read(self):
        return (self._x + self._w + self._b) * self.unit

    @property
    def output_bytes_written(self):
        return self._y * self.unit

    @property
    def output_accumulation_depth(self):
        return self._depth

    # grad_input from grad_output and weight
    @property
    def grad_input_macs(self):
        return self._x * self._depth

    @property
    def grad_input_bytes_read(self):
        return (self._y + self._w) * self.unit

    @property
    def grad_input_bytes_written(self):
        return self._x * self.unit

    @property
    def grad_input_accumulation_depth(self):
        return self._depth

    # grad_weight from input and grad_output
    @property
    def grad_weight_macs(self):
        return self._x * self._depth

    @property
    def grad_weight_bytes_read(self):
        return (self._y + self._x) * self.unit

    @property
    def grad_weight_bytes_written(self):
        return self._w * self.unit

    @property
    def grad_weight_accumulation_depth(self):
        return self.params.n * self.params.h * self.params.w

    # grad_bias from grad_output
    @property
    def grad_bias_macs(self):
        return self._y / 2

    @property
    def grad_bias_bytes_read(self):
        return self._y * self.unit

    @property
    def grad_bias_bytes_written(self):
        return self._b * self.unit

    @property
    def grad_bias_accumulation_depth(self):
        return self.params.n * self.params.h * self.params.w
