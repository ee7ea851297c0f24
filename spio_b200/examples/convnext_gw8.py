"""A ConvNeXt-T-style network whose 7x7 depthwise convolutions are replaced by 3x3 grouped
convolutions of group width 8 -- the layers ``spio_b200.transform.transform`` swaps for
``Conv2dGw8``.

Widths 96/192/384/768, depths 3/3/9/3; each block is gw8 conv -> LayerNorm -> 1x1 expand 4x ->
GELU -> 1x1 project -> residual.  The definition is plain ``torch.nn`` and fx-traceable; the
reference relies on timm for its models (scripts/profile_block.py), which is not a dependency
here.

    python -m spio_b200.examples.convnext_gw8 --batch 256 --steps 5     # times one train step
"""

from __future__ import annotations

import argparse
import time
from typing import Sequence

import torch
from torch import nn


class LayerNorm2d(nn.Module):
    """LayerNorm over the channel dimension of an NCHW tensor."""

    def __init__(self, channels: int, eps: float = 1e-6):
        super().__init__()
        self.norm = nn.LayerNorm(channels, eps=eps)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.norm(x.permute(0, 2, 3, 1)).permute(0, 3, 1, 2)


class Block(nn.Module):
    def __init__(self, dim: int):
        super().__init__()
        self.conv = nn.Conv2d(dim, dim, kernel_size=3, padding=1, groups=dim // 8)  # group width 8
        self.norm = LayerNorm2d(dim)
        self.expand = nn.Conv2d(dim, 4 * dim, kernel_size=1)
        self.act = nn.GELU()
        self.project = nn.Conv2d(4 * dim, dim, kernel_size=1)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x + self.project(self.act(self.expand(self.norm(self.conv(x)))))


class ConvNeXtGw8(nn.Module):
    def __init__(self, widths: Sequence[int] = (96, 192, 384, 768), depths: Sequence[int] = (3, 3, 9, 3),
                 num_classes: int = 1000, in_chans: int = 3):
        super().__init__()
        layers = [nn.Conv2d(in_chans, widths[0], kernel_size=4, stride=4), LayerNorm2d(widths[0])]
        for i, (w, d) in enumerate(zip(widths, depths)):
            if i > 0:
                layers += [LayerNorm2d(widths[i - 1]), nn.Conv2d(widths[i - 1], w, kernel_size=2, stride=2)]
            layers += [Block(w) for _ in range(d)]
        self.features = nn.Sequential(*layers)
        self.pool = nn.AdaptiveAvgPool2d(1)
        self.head_norm = nn.LayerNorm(widths[-1])
        self.head = nn.Linear(widths[-1], num_classes)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.pool(self.features(x)).flatten(1)
        return self.head(self.head_norm(x))


def swap_layernorm(model: nn.Module) -> int:
    """Replace every channel LayerNorm of the network (the LayerNorm2d wrapper above) by the
    fused ``spio_b200.layers.LayerNorm2d``; returns how many were replaced."""
    from spio_b200.layers import LayerNorm2d as FusedLayerNorm2d

    count = 0
    for parent in model.modules():
        for name, child in list(parent.named_children()):
            if isinstance(child, LayerNorm2d) and FusedLayerNorm2d.match(child.norm):
                setattr(parent, name, FusedLayerNorm2d.from_torch_module(child.norm))
                count += 1
    return count


def train_step(model: nn.Module, images: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
    """Forward + backward under fp16 autocast; returns the loss."""
    with torch.autocast("cuda", dtype=torch.float16):
        loss = nn.functional.cross_entropy(model(images).float(), labels)
    loss.backward()
    return loss.detach()


def main() -> None:
    from spio_b200.transform._transform import _transform

    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=5)
    args = ap.parse_args()
    torch.manual_seed(1234 + 4)
    dev = torch.device("cuda")
    model = ConvNeXtGw8().to(dev).to(memory_format=torch.channels_last)
    images = torch.randn(args.batch, 3, 224, 224, device=dev).contiguous(memory_format=torch.channels_last)
    labels = torch.randint(0, 1000, (args.batch,), device=dev)
    import copy

    fast, replaced = _transform(model)
    with_ln = copy.deepcopy(model)
    n_ln = swap_layernorm(with_ln)          # before tracing: transform keeps the fused modules
    fused, _ = _transform(with_ln)
    for name, net in (("torch / cuDNN grouped conv", model), (f"spio_b200 ({replaced} layers swapped)", fast),
                      (f"spio_b200 ({replaced} convs + {n_ln} LayerNorm2d swapped)", fused)):
        for _ in range(2):
            net.zero_grad(set_to_none=True)
            train_step(net, images, labels)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            net.zero_grad(set_to_none=True)
            loss = train_step(net, images, labels)
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) / args.steps * 1e3
        print(f"{name}: {ms:.1f} ms / train step at batch {args.batch} (loss {float(loss):.4f})", flush=True)


if __name__ == "__main__":
    main()
