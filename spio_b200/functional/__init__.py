"""Functional operators (the names the reference exports from spio.functional)."""

from .conv2d_gw8_function import conv2d_gw8, conv2d_gw8_backward_op
