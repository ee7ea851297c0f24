"""Memory-format helpers: the kernels take 4-D tensors in channels_last (NHWC) order
(reference: spio/util/tensor_format.py:8-17, spio/util/memory_format.py:32-38)."""

from __future__ import annotations

import torch


def _one_channels_last(t):
    if t is None or t.dim() != 4:
        return t
    return t.contiguous(memory_format=torch.channels_last)


def to_channels_last(*args):
    """Each 4-D tensor in channels_last layout (a copy only if it is not already)."""
    out = tuple(_one_channels_last(a) for a in args)
    return out[0] if len(out) == 1 else out


def check_channels_last(args) -> None:
    """Assert every 4-D tensor argument is laid out channels_last."""
    for a in args:
        if a is not None and hasattr(a, "dim") and a.dim() == 4:
            assert a.is_contiguous(memory_format=torch.channels_last), (
                f"Tensor of shape {tuple(a.shape)} with strides {a.stride()} is not channels_last")


def get_device_ordinal(device) -> int:
    dev = torch.device(device)
    if dev.index is not None:
        return dev.index
    return torch.cuda.current_device() if dev.type == "cuda" else 0
