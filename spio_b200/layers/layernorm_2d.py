"""``LayerNorm2d``: LayerNorm over the channels of an NCHW tensor, backed by the
``spio::layernorm_2d`` operator (fp16 channels_last data on a CUDA device; use it under
``torch.autocast("cuda", dtype=torch.float16)`` for fp32 models)."""

from __future__ import annotations

import torch
from torch import nn

from ..functional.layernorm_2d_function import layernorm_2d


class LayerNorm2d(nn.Module):
    def __init__(self, num_channels: int, eps: float = 1e-6, elementwise_affine: bool = True,
                 device=None, dtype=torch.float32):
        super().__init__()
        if num_channels % 8 != 0 or num_channels > 1024:
            raise ValueError("LayerNorm2d needs a multiple of 8 channels, at most 1024")
        self.num_channels = num_channels
        self.eps = eps
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(num_channels, device=device, dtype=dtype))
            self.bias = nn.Parameter(torch.zeros(num_channels, device=device, dtype=dtype))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    @staticmethod
    def match(module: nn.Module) -> bool:
        """True for an ``nn.LayerNorm`` over one dimension that this layer can replace when
        it is applied to the channel dimension of an image tensor."""
        return (isinstance(module, nn.LayerNorm) and len(module.normalized_shape) == 1
                and module.normalized_shape[0] % 8 == 0 and module.normalized_shape[0] <= 1024)

    @staticmethod
    def from_torch_module(module: nn.LayerNorm) -> "LayerNorm2d":
        """Same parameters (shared, not copied) as the given ``nn.LayerNorm``."""
        ln = LayerNorm2d(module.normalized_shape[0], eps=module.eps,
                         elementwise_affine=module.elementwise_affine)
        if module.elementwise_affine:
            ln.weight = module.weight
            ln.bias = module.bias
        return ln

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return layernorm_2d(x, self.weight, self.bias, self.eps)

    def extra_repr(self) -> str:
        return f"{self.num_channels}, eps={self.eps}, elementwise_affine={self.weight is not None}"
