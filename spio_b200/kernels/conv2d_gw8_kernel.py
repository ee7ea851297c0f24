"""Forward / input-gradient kernel family: tile configurations and the kernel factory.

Counterpart of the reference's spio/kernels/conv2d_gw8_kernel.py:30-238.  A configuration
there fixes (groups per CTA, block_p, block_n) of a one-tile-per-CTA kernel; here the
kernel is persistent and streams row pairs through a shared-memory ring, so a
configuration fixes the warp mapping and the ring instead:

    wpg  compute warps per channel group        tpw  8-pixel x 2-row tiles per warp
    pps  row pairs per ring slot                 ncb  8-pixel column blocks per column tile
    nb   images per ring slot                    ns   ring slots
    nob  output staging buffers                   engine  1 = warp-level mma.sync kernel,
                                                          2 = tcgen05 kernel (tensor memory)

A zero means "let the launch planner choose".  Engine 2 exists for filters up to 3 x 3; it
takes ncb, ns and nob only.
"""

from __future__ import annotations

import ctypes
import os
from dataclasses import asdict, dataclass, replace
from typing import Iterator, List

from .. import _clib
from ..util.math import divup
from .conv2d_gw8_params import Conv2dGw8Params
from .conv2d_stats import Conv2dStats
from .kernel import shape_of
from .kernel_factory import KernelFactory


@dataclass(frozen=True)
class Conv2dGw8Config:
    wpg: int = 0
    tpw: int = 0
    pps: int = 0
    ncb: int = 0
    nb: int = 0
    ns: int = 0
    nob: int = 0
    engine: int = 0

    def as_tune(self) -> dict:
        return asdict(self)


def compiled_variants(r: int, s: int) -> List[tuple]:
    """(wpg, tpw, pps) triples compiled into the library for an r x s filter."""
    lib = _clib.load()
    out = []
    vr, vs, vw, vt, vp = (ctypes.c_int() for _ in range(5))
    for i in range(lib.spio_conv2d_gw8_num_variants()):
        lib.spio_conv2d_gw8_variant(i, ctypes.byref(vr), ctypes.byref(vs), ctypes.byref(vw),
                                    ctypes.byref(vt), ctypes.byref(vp))
        if (vr.value, vs.value) == (r, s):
            out.append((vw.value, vt.value, vp.value))
    return out


# Configurations with an explicit ring depth stay within the 196 KiB shared-memory configuration
# of the SM: the 228 KiB one leaves 28 KiB of L1, too little for the kernels' spilled loop
# invariants, and it is sticky across dependent launches (the planner's own choice, ns = 0,
# follows the same rule).
SMEM_SOFT_CAP = 194 * 1024


def plan_is_valid(kind: int, params, tune: dict, device_attr, smem_cap: int = 0) -> bool:
    lib = _clib.load()
    info = _clib.PlanInfo()
    t = _clib.make_tune(tune)
    rc = lib.spio_conv2d_gw8_plan_for(kind, ctypes.byref(shape_of(params)), ctypes.byref(t),
                                      device_attr.multiprocessor_count,
                                      device_attr.max_shared_memory_per_block_optin,
                                      ctypes.byref(info))
    return rc == 0 and (smem_cap <= 0 or info.smem_bytes <= smem_cap)


def enumerate_tiles(params, out_w: int, wpg: int, tpw: int, forward: bool = False) -> Iterator[tuple]:
    """(ncb, nb) candidates: (0, 0) = the launch planner's own choice, then the width cut into
    1..4 column tiles; several images per slot
    only when one tile spans the whole width.  ncb counts 8-pixel column blocks.  The
    weight-gradient kernel holds wpg * tpw tiles of 8 pixels; the forward kernel holds
    wpg * ceil(tpw / 2) blocks of 16 pixels and its column tile is at least 16 pixels wide, except
    that images at most 8 pixels wide may be paired: ncb = 1 and an even nb put two images into
    the two halves of every block."""
    max_tiles = wpg * ((tpw + 1) // 2) if forward else wpg * tpw
    need = (lambda ncb: divup(max(ncb, 2), 2)) if forward else (lambda ncb: ncb)
    col_blocks = divup(out_w, 8)
    seen = set()
    yield 0, 0  # always plannable: wide images with few tiles per warp need more column tiles than tried below
    if forward and col_blocks == 1:
        # images at most 8 pixels wide: two images share a 16-pixel block (ncb = 1, nb even)
        nb = 2
        while nb <= 2 * max_tiles and nb <= params.n:
            yield 1, nb
            nb *= 2
    for n_ct in range(1, 5):
        ncb = max(divup(col_blocks, n_ct), 2 if forward else 1)
        if need(ncb) > max_tiles or ncb in seen:
            continue
        seen.add(ncb)
        yield ncb, 1
        if ncb >= col_blocks:
            nb = 2
            while nb * need(ncb) <= max_tiles and nb <= params.n:
                yield ncb, nb
                nb *= 2


def _get_configs(params: Conv2dGw8Params, device_attr, igrad: bool = False) -> Iterator[Conv2dGw8Config]:
    kind = _clib.DGRAD if igrad else _clib.FPROP
    out_w = params.w if igrad else params.q
    for wpg, tpw, pps in compiled_variants(params.r, params.s):
        for ncb, nb in enumerate_tiles(params, out_w, wpg, tpw, forward=True):
            for ns in (0, 3, 4, 6):
                for nob in (2, 3):
                    cfg = Conv2dGw8Config(wpg=wpg, tpw=tpw, pps=pps, ncb=ncb, nb=nb, ns=ns, nob=nob)
                    if plan_is_valid(kind, params, cfg.as_tune(), device_attr, SMEM_SOFT_CAP if ns else 0):
                        yield cfg
    if params.r <= 3 and params.s <= 3 and os.environ.get("SPIO_TUNE_TCGEN05", "0") == "1":
        # the tcgen05 kernel: column tiles of up to 64 - (s - 1) pixels, ring depth, staging buffers.
        # It lost on every measured shape, so it is enumerated only on request (SPIO_TUNE_TCGEN05=1);
        # an explicit Conv2dGw8Config(engine=2) still selects it.
        for n_ct in range(1, 4):
            ncb = divup(divup(out_w, 8), n_ct)
            for ns in (0, 4, 6):
                for nob in (2, 3):
                    cfg = Conv2dGw8Config(engine=2, ncb=ncb, ns=ns, nob=nob)
                    if plan_is_valid(kind, params, cfg.as_tune(), device_attr):
                        yield cfg


def _cap_ring(params: Conv2dGw8Params, config: Conv2dGw8Config, device_attr, igrad: bool = False):
    """Tuning-table entries measured one kernel at a time may ask for a ring above the soft
    cap; in a chain of dependent launches that costs more than the deeper ring gains, so the
    depth goes back to the planner (which stops at the cap)."""
    if config.engine == 2 or not config.ns:
        return config
    kind = _clib.DGRAD if igrad else _clib.FPROP
    if plan_is_valid(kind, params, config.as_tune(), device_attr, SMEM_SOFT_CAP):
        return config
    capped = replace(config, ns=0)
    return capped if plan_is_valid(kind, params, capped.as_tune(), device_attr) else config


def _get_kernel_name(igrad: bool = False) -> str:
    return "spio_conv2d_gw8_dgrad" if igrad else "spio_conv2d_gw8_fprop"


conv2d_gw8_kernel_factory = KernelFactory(
    Conv2dGw8Params,
    Conv2dGw8Config,
    Conv2dStats,
    kernel_name=_get_kernel_name,
    configs=_get_configs,
    perf_model_skip_params=["group_width", "stride"],
    fixup=_cap_ring,
)
