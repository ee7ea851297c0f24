"""Operation and byte counts of a kernel, summed over the outputs it produces.

Interface of the reference's ``Stats`` base class (spio/kernels/stats.py:8-67): a
subclass defines ``<output>_macs``, ``<output>_bytes_read``, ``<output>_bytes_written``
and ``<output>_accumulation_depth`` for every output name it knows.
"""

from __future__ import annotations

from typing import List, Sequence, Union


class Stats:
    def __init__(self, params=None, unit: int = 2, output_names: Union[str, Sequence[str], None] = None):
        self.params = params
        self.unit = unit  # bytes per tensor element
        self.output_names = [output_names] if isinstance(output_names, str) else output_names

    def _total(self, suffix: str):
        return sum(getattr(self, f"{name}_{suffix}") for name in self.output_names)

    @property
    def macs(self):
        return self._total("macs")

    @property
    def bytes_read(self):
        return self._total("bytes_read")

    @property
    def bytes_written(self):
        return self._total("bytes_written")

    @property
    def bytes(self):
        return self.bytes_read + self.bytes_written

    @property
    def op_byte(self) -> float:
        return 2.0 * self.macs / self.bytes

    @property
    def accumulation_depths(self) -> List[int]:
        return [getattr(self, f"{name}_accumulation_depth") for name in self.output_names]
