"""Loads and launches the REFERENCE's own gw8 kernels (compiled for sm_100a into ``oracle/_ref/`` by
``oracle/build_ref_kernels.py``).  TEST INFRASTRUCTURE ONLY: used by the tests as a second oracle
(this package's kernels against the reference's kernels on the same inputs) and by ``bench.py`` as
the incumbent arm.  Nothing under ``spio_b200/`` imports this module.

The cubins are loaded with this package's driver-API module loader and launched as the reference's
``Kernel.launch`` launches them (spio/kernels/kernel.py:135-154, spio/cuda/driver.pyx:171-208): a
one-dimensional grid and block from the kernel's own launch parameters, no dynamic shared memory,
plain tensor pointers in the order

    fprop (output, input, weight, bias | NULL)      dgrad (grad_input, grad_output, weight, NULL)
    wgrad (grad_weight fp32, ZERO-FILLED by the caller; input; grad_output)

All tensors are channels_last, fp16 except grad_weight.  The kernels are specialised per layer
shape, so a cubin runs exactly the shape recorded in the manifest; ``kernels_for`` refuses any other.
"""

from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, List, Optional

REF_DIR = Path(__file__).resolve().parent / "_ref"


def available() -> bool:
    return (REF_DIR / "manifest.json").exists()


def manifest() -> List[dict]:
    if not available():
        return []
    return json.loads((REF_DIR / "manifest.json").read_text())["kernels"]


class RefKernel:
    def __init__(self, row: dict):
        self.row = row
        self.kind = row["kind"]
        self.shape = row["shape"]
        self.config = row["config"]
        self.module = None
        self.function = None

    def load(self) -> "RefKernel":
        from spio_b200.cuda.driver import Module

        if self.function is None:
            self.module = Module()
            self.module.load_data((REF_DIR / self.row["file"]).read_bytes())
            self.function = self.module.get_function(self.row["function"])
        return self

    def unload(self) -> None:
        self.function = None
        if self.module is not None:
            self.module.unload()
            self.module = None

    def check(self, tensors) -> None:
        """The cubin is compiled for one shape: refuse anything else before it reaches the GPU."""
        import torch

        s = self.shape
        act = (s["n"], s["c"], s["h"], s["w"])
        wgt = (s["c"], 8, s["r"], s["s"])
        want = {"fprop": [act, act, wgt], "dgrad": [act, act, wgt], "wgrad": [wgt, act, act]}[self.kind]
        dtypes = {"fprop": [torch.float16] * 3, "dgrad": [torch.float16] * 3,
                  "wgrad": [torch.float32, torch.float16, torch.float16]}[self.kind]
        for t, shape, dt in zip(tensors, want, dtypes):
            if tuple(t.shape) != shape or t.dtype != dt or not t.is_cuda:
                raise ValueError(f"reference kernel {self.row['function']} takes {shape} {dt}, got {tuple(t.shape)} {t.dtype}")
            if not t.is_contiguous(memory_format=torch.channels_last):
                raise ValueError("reference kernels take channels_last tensors")

    def __call__(self, *tensors) -> None:
        """fprop: (y, x, w, bias | None); dgrad: (dx, dy, w); wgrad: (dw zero-filled, x, dy)."""
        self.check([t for t in tensors[:3]])
        args = list(tensors)
        if self.kind == "fprop" and len(args) == 3:
            args.append(None)
        if self.kind == "dgrad":
            args = args[:3] + [None]
        self.function.launch(self.row["grid"], self.row["block"], args, shared_mem_bytes=self.row["shared_mem_bytes"])

    def __repr__(self) -> str:
        return f"{self.row['function']} {self.config}"


def kernels_for(kind: str, n: int, c: int, h: int, w: int, r: int = 3, s: int = 3, pad: int = 1) -> List[RefKernel]:
    """The reference's kernels compiled for exactly this layer shape (one per configuration)."""
    want = {"n": n, "c": c, "h": h, "w": w, "r": r, "s": s, "pad_h": pad, "pad_w": pad}
    return [RefKernel(row) for row in manifest() if row["kind"] == kind and row["shape"] == want]


def shapes() -> List[Dict[str, int]]:
    seen, out = set(), []
    for row in manifest():
        key = tuple(sorted(row["shape"].items()))
        if key not in seen:
            seen.add(key)
            out.append(row["shape"])
    return out
