"""Weight-gradient kernel family: tile configurations and the kernel factory.

Counterpart of the reference's spio/kernels/conv2d_gw8_wgrad_kernel.py:27-285.  The
fields have the meaning given in conv2d_gw8_kernel.py; the weight-gradient kernel has no
output staging buffers, and a ring slot holds an input box and an output-gradient box.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass
from typing import Iterator

from .. import _clib
from .conv2d_gw8_kernel import SMEM_SOFT_CAP, compiled_variants, enumerate_tiles, plan_is_valid
from .conv2d_gw8_params import Conv2dGw8Params
from .conv2d_stats import Conv2dStats
from .kernel_factory import KernelFactory


@dataclass(frozen=True)
class Conv2dGw8WgradConfig:
    wpg: int = 0
    tpw: int = 0
    pps: int = 0
    ncb: int = 0
    nb: int = 0
    ns: int = 0

    def as_tune(self) -> dict:
        return asdict(self)


def _get_configs(params: Conv2dGw8Params, device_attr) -> Iterator[Conv2dGw8WgradConfig]:
    for wpg, tpw, pps in compiled_variants(params.r, params.s):
        for ncb, nb in enumerate_tiles(params, params.q, wpg, tpw):
            for ns in (0, 2, 3, 4):
                cfg = Conv2dGw8WgradConfig(wpg=wpg, tpw=tpw, pps=pps, ncb=ncb, nb=nb, ns=ns)
                if plan_is_valid(_clib.WGRAD, params, cfg.as_tune(), device_attr, SMEM_SOFT_CAP if ns else 0):
                    yield cfg


conv2d_gw8_wgrad_kernel_factory = KernelFactory(
    Conv2dGw8Params,
    Conv2dGw8WgradConfig,
    Conv2dStats,
    kernel_name="spio_conv2d_gw8_wgrad",
    configs=_get_configs,
    perf_model_skip_params=["group_width", "stride"],
)
