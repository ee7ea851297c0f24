"""Effective bandwidth of the three gw8 kernels against batch size, as a table.

The reference measures this by profiling a ConvFirst block at batch 32 ... 256 and plotting
algorithmic bytes / kernel time per kernel (scripts/profile_blocks.bash:4-5,
scripts/plot_kernel_bench.py:430-435); here the kernels the factories choose for each shape are
timed directly, in chains of back-to-back launches over operand sets larger than the L2 cache, and
the result is printed as text (and optionally written as CSV).

    python -m spio_b200.kernels.bench_kernels --channels 64 --hw 56 --batches 32,64,128,256
"""

from __future__ import annotations

import argparse
import csv
import sys
from typing import Optional

import torch

from ..cuda.driver import get_device_attributes
from .autotune import KERNELS, make_operand_sets, time_kernel
from .conv2d_gw8_params import Conv2dGw8Params
from .conv2d_stats import Conv2dStats
from .kernel import device_status


def measure(params: Conv2dGw8Params, device: torch.device, warm: bool = False) -> dict:
    """{kernel: (microseconds, GB/s, configuration)} with the configuration the factory selects.
    ``warm``: two operand sets instead of four L2 sizes' worth, so that small layers stay in the L2
    cache from launch to launch (the situation inside a network, and the reason the reference's
    RTX 4090 figure exceeds the DRAM bandwidth at small batch)."""
    attr = get_device_attributes(device.index or 0)
    nbytes = Conv2dStats(params, output_names="output").bytes
    out = {}
    for name, (factory, kwargs) in sorted(KERNELS.items()):
        kernel = factory.get_kernel(params, device, **kwargs)
        sets = make_operand_sets(name, params, device, min_bytes=1 if warm else 4 * attr.l2_cache_size)
        ms = time_kernel(kernel, sets, reps=5)
        out[name.replace("spio_conv2d_gw8_", "")] = (ms * 1e3, nbytes / ms / 1e6, kernel.config)
        del sets
        torch.cuda.empty_cache()
    return out


def main(argv: Optional[list] = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--channels", type=int, default=64)
    ap.add_argument("--hw", type=int, default=56)
    ap.add_argument("--filter", type=int, default=3)
    ap.add_argument("--batches", default="32,64,96,128,160,192,224,256")
    ap.add_argument("--warm", action="store_true", help="two operand sets only: small layers stay in the L2 cache")
    ap.add_argument("--csv", default=None, help="also write the rows to this file")
    args = ap.parse_args(argv)
    device = torch.device("cuda", torch.cuda.current_device())
    rows = []
    print(f"{'batch':>6} | " + " | ".join(f"{k:>22}" for k in ("dgrad", "fprop", "wgrad")))
    for n in (int(t) for t in args.batches.split(",")):
        params = Conv2dGw8Params(n=n, c=args.channels, h=args.hw, w=args.hw, r=args.filter, s=args.filter,
                                 padding=args.filter // 2)
        res = measure(params, device, warm=args.warm)
        print(f"{n:>6} | " + " | ".join(f"{res[k][0]:8.1f} us {res[k][1]:7.0f} GB/s" for k in ("dgrad", "fprop", "wgrad")),
              flush=True)
        for k, (us, gbs, cfg) in res.items():
            rows.append({"batch": n, "kernel": k, "us": round(us, 2), "GBps": round(gbs, 1), "config": str(cfg)})
    if device_status() != 0:
        sys.exit("a kernel reported a wait time-out")
    if args.csv:
        with open(args.csv, "w", newline="") as fh:
            wr = csv.DictWriter(fh, fieldnames=["batch", "kernel", "us", "GBps", "config"])
            wr.writeheader()
            wr.writerows(rows)


if __name__ == "__main__":
    main()
