"""Device attributes the kernel planner and the configuration spaces depend on.

Counterpart of ``get_device_attributes`` in the reference's Cython driver module
(spio/cuda/driver.pyx:275-330); here the values come from the CUDA runtime through
torch, and a fixed B200 record is available for planning on machines without a GPU.
"""

from __future__ import annotations

from dataclasses import dataclass
from functools import lru_cache
from typing import Tuple


@dataclass(frozen=True)
class DeviceAttributes:
    name: str = "NVIDIA B200"
    multiprocessor_count: int = 148
    l2_cache_size: int = 132120576
    compute_capability: Tuple[int, int] = (10, 0)
    max_shared_memory_per_block_optin: int = 232448
    max_shared_memory_per_block: int = 49152
    num_partitions_per_sm: int = 4

    @property
    def arch(self) -> str:
        major, minor = self.compute_capability
        return f"sm_{major}{minor}" + ("a" if major >= 9 else "")


# What `get_device_attributes` returns on the B200s this package targets.
B200_ATTRIBUTES = DeviceAttributes()


@lru_cache(maxsize=None)
def get_device_attributes(device_ordinal: int = 0) -> DeviceAttributes:
    import torch

    if not torch.cuda.is_available():
        raise ValueError("CUDA error: no CUDA device is available")
    prop = torch.cuda.get_device_properties(device_ordinal)
    return DeviceAttributes(
        name=prop.name,
        multiprocessor_count=prop.multi_processor_count,
        l2_cache_size=getattr(prop, "L2_cache_size", 0),
        compute_capability=(prop.major, prop.minor),
        max_shared_memory_per_block_optin=getattr(prop, "shared_memory_per_block_optin", 232448),
        max_shared_memory_per_block=getattr(prop, "shared_memory_per_block", 49152),
        num_partitions_per_sm=4,
    )
