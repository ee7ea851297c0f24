"""Key of a cached kernel: the device it was loaded for and the problem shape
(reference: spio/kernels/kernel_key.py:13-18)."""

from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class KernelKey:
    device_ordinal: int
    params: Any
