"""Layers (the names the reference exports from spio.layers)."""

from .conv2d_gw8 import Conv2dGw8
from .make import make_conv2d
from .layernorm_2d import LayerNorm2d
