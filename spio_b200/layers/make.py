"""Factory over all layer classes of the package (reference: spio/layers/make.py)."""

from .conv2d_gw8 import Conv2dGw8


def make_conv2d(*args, **kwargs):
    """A layer implementing ``nn.Conv2d(*args, **kwargs)``, or None when no layer of this
    package supports those arguments."""
    return Conv2dGw8.make(*args, **kwargs)
