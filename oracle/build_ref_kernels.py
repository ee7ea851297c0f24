"""Compiles the REFERENCE's own gw8 kernels for sm_100a into ``oracle/_ref/``.  TEST INFRASTRUCTURE ONLY.

    python oracle/build_ref_kernels.py /path/to/andravin-spio-checkout

The reference implements this path only as CUDA kernels that its Python generators specialise per
(layer shape, tile configuration) and NVRTC compiles; it has no CPU build.  Its generators and its
NVRTC wrapper run without a GPU, so this script imports them FROM THE CHECKOUT WHERE IT LIES (nothing
is copied into this repository), generates the per-shape ``types.h`` for a bounded set of the
reference's own tile configurations, compiles ``spio/src/conv2d_gw8.cu`` / ``conv2d_gw8_wgrad.cu``
against it with ``-arch=sm_100a`` and writes

    oracle/_ref/<kernel name>__<i>.cubin        one cubin per (kernel, shape, configuration)
    oracle/_ref/manifest.json                   kernel name, shape, configuration, grid, block

``oracle/ref_kernels.py`` loads those cubins on the GPU box (where the checkout does not exist)
through this package's driver-API module loader and launches them exactly as the reference's
``Kernel.launch`` does (spio/kernels/kernel.py:135-154: 1-D grid and block, no dynamic shared
memory, plain tensor pointers).  They serve two purposes: a parity check of this package's kernels
against the reference's kernels themselves, and the incumbent arm of the benchmark.

Four small stand-ins make the reference importable here: ``importlib_resources`` and ``appdirs``
(wheels that are not installed; trivial shims over the standard library), ``xgboost`` (only its
performance-model code needs it; configurations are given explicitly, as the reference's own tests
do, spio/src_tests/run_test.py:51-57) and ``spio.cuda.driver`` (a Cython extension that needs
libcuda; only ``DeviceAttributes`` is used, filled with the B200's published limits).
"""

from __future__ import annotations

import dataclasses
import importlib
import importlib.resources
import json
import os
import sys
import types
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

OUT = Path(__file__).resolve().parent / "_ref"

# (n, c, h, w): 3x3, stride 1, pad 1, no bias -- the batch sweep of the 64-channel 56x56 layer and the
# channel / resolution ladder, the shapes the benchmark reports
SHAPES = [(128, 64, 56, 56), (256, 64, 56, 56), (512, 64, 56, 56), (2048, 64, 56, 56),
          (256, 128, 56, 56), (256, 256, 28, 28), (256, 512, 14, 14), (256, 768, 7, 7),
          (8, 64, 32, 32), (6, 72, 19, 23)]
MAX_FWD_CONFIGS = 6     # per shape and mode, spread over the reference's configuration space
MAX_WGRAD_CONFIGS = 10


def install_stand_ins() -> type:
    ir = types.ModuleType("importlib_resources")
    ir.files = importlib.resources.files
    ira = types.ModuleType("importlib_resources.abc")
    ira.Traversable = object
    sys.modules["importlib_resources"], sys.modules["importlib_resources.abc"] = ir, ira
    ad = types.ModuleType("appdirs")
    ad.user_cache_dir = lambda name: os.path.join("/tmp", name)
    sys.modules["appdirs"] = ad
    xg = types.ModuleType("xgboost")
    xg.Booster = xg.DMatrix = object
    sys.modules["xgboost"] = xg

    drv = types.ModuleType("spio.cuda.driver")

    @dataclasses.dataclass(frozen=True)
    class DeviceAttributes:
        multiprocessor_count: int = 148
        l2_cache_size: int = 126 * 1024 * 1024
        name: str = "NVIDIA B200"
        compute_capability: tuple = (10, 0)
        max_shared_memory_per_block_optin: int = 232448
        max_shared_memory_per_block: int = 48 * 1024
        num_partitions_per_sm: int = 4

    @dataclasses.dataclass(frozen=True)
    class FunctionAttributes:
        max_dynamic_shared_memory_size: int = None
        preferred_shared_memory_carveout: int = None

    class PrimaryContextGuard:
        def set_device(self, _device):
            pass

    drv.DeviceAttributes, drv.FunctionAttributes = DeviceAttributes, FunctionAttributes
    drv.PrimaryContextGuard, drv.init = PrimaryContextGuard, (lambda: None)
    drv.Module = drv.Function = object
    drv.get_device_attributes = lambda _i=0: DeviceAttributes()
    sys.modules["spio.cuda.driver"] = drv
    return DeviceAttributes


def spread(items, limit):
    items = list(items)
    if len(items) <= limit:
        return items
    step = len(items) / limit
    return [items[int(i * step)] for i in range(limit)]


def main(root: Path) -> None:
    os.environ.setdefault("SPIO_WORKERS", "1")
    sys.path.insert(0, str(root))
    device_attributes = install_stand_ins()
    from spio.compiler.compile import compile_cuda
    from spio.kernels import (Conv2dGw8Config, Conv2dGw8Params, Conv2dGw8WgradConfig, conv2d_gw8_kernel_factory,
                              conv2d_gw8_wgrad_kernel_factory)

    da = device_attributes()
    OUT.mkdir(parents=True, exist_ok=True)
    jobs = []
    for n, c, h, w in SHAPES:
        params = Conv2dGw8Params(n=n, c=c, h=h, w=w, padding=1, r=3, s=3)
        # configurations in the neighbourhood the reference's examples use (8 groups per CTA), its
        # own defaults first
        fwd = [Conv2dGw8Config(groups=8, block_p=16 if params.p >= 16 else params.p, block_n=1)]
        fwd += [cfg for cfg in conv2d_gw8_kernel_factory.configs(params, da) if cfg.groups == 8 and cfg not in fwd
                and cfg.block_p >= 4]
        wgr = [cfg for cfg in conv2d_gw8_wgrad_kernel_factory.configs(params, da)
               if cfg.groups == 8 and cfg.warp_s == 3 and cfg.block_h >= 4 and cfg.block_n_iters >= 2]
        for kind, factory, configs, kwargs in (
                ("fprop", conv2d_gw8_kernel_factory, [fwd[0]] + spread(fwd[1:], MAX_FWD_CONFIGS - 1), {}),
                ("dgrad", conv2d_gw8_kernel_factory, [fwd[0]] + spread(fwd[1:], MAX_FWD_CONFIGS - 1), {"igrad": True}),
                ("wgrad", conv2d_gw8_wgrad_kernel_factory, spread(wgr, MAX_WGRAD_CONFIGS), {})):
            for i, cfg in enumerate(configs):
                jobs.append((kind, factory, params, cfg, kwargs, i))

    def build(job):
        kind, factory, params, cfg, kwargs, i = job
        try:
            kernel = factory.make_kernel(params, cfg, da, **kwargs)
            src, header_dict, src_module, include_module = kernel.compiler_args
            cubin = compile_cuda(importlib.resources.files(src_module).joinpath(src),
                                 includes=[str(importlib.resources.files(include_module))], arch="sm_100a",
                                 header_dict=header_dict)
        except Exception as exc:  # a configuration the reference's own checks reject
            return {"kind": kind, "error": f"{type(exc).__name__}: {str(exc)[:120]}", "config": repr(cfg)}
        launch = kernel.kernel_spec.launch_params
        grid = launch.grid if isinstance(launch.grid, int) else launch.grid[0]
        block = launch.block if isinstance(launch.block, int) else launch.block[0]
        name = f"{kernel.kernel_name}__{i}.cubin"
        (OUT / name).write_bytes(bytes(cubin))
        return {"kind": kind, "file": name, "function": kernel.kernel_name, "config": dataclasses.asdict(cfg),
                "grid": int(grid), "block": int(block), "shared_mem_bytes": int(launch.shared_mem_bytes or 0),
                "shape": {"n": params.n, "c": params.c, "h": params.h, "w": params.w, "r": params.r, "s": params.s,
                          "pad_h": params.padding_h, "pad_w": params.padding_w}}

    with ThreadPoolExecutor(max_workers=os.cpu_count() or 2) as pool:
        rows = list(pool.map(build, jobs))
    good = [r for r in rows if "file" in r]
    (OUT / "manifest.json").write_text(json.dumps({"kernels": good, "rejected": [r for r in rows if "error" in r],
                                                   "arch": "sm_100a"}, indent=1) + "\n")
    print(f"compiled {len(good)} reference kernels into {OUT} ({len(rows) - len(good)} configurations rejected)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python oracle/build_ref_kernels.py <path of the andravin/spio checkout>")
    main(Path(sys.argv[1]))
