"""Grid, block and dynamic shared memory of one launch
(reference: spio/kernels/launch_params.py)."""

from dataclasses import dataclass


@dataclass(frozen=True)
class LaunchParams:
    grid: int
    block: int
    shared_mem_bytes: int = 0
