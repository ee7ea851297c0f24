"""Functional operators (the names the reference exports from spio.functional)."""

from .conv2d_gw8_function import (conv2d_gw8, conv2d_gw8_backward_op, get_grad_weight_dtype,
                                  set_grad_weight_dtype)
from .layernorm_2d_function import layernorm_2d, layernorm_2d_op, layernorm_2d_backward_op
