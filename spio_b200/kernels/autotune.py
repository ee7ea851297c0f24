"""Measure tile configurations on the device, keep the best per layer shape, train the model.

The reference collects (kernel, params, config, latency) rows by running a model under
torch.profiler with random configuration overlays and trains one XGBoost regressor per kernel
from them (scripts/profile_block.py:551-701, scripts/train_performance_model.py:46-142).  Here
each configuration of a kernel family's configuration space is timed directly with CUDA events
on operands larger than the L2 cache; the fastest goes into the tuning table that
``PerformanceModelCache`` consults first, and all rows can be fitted by the small
gradient-boosted-tree model in ``gbt_model.py`` for shapes that were never measured.

    python -m spio_b200.kernels.autotune --shape 256,64,56,56 --shape 256,128,56,56 \
        --out spio_b200/kernels/perf_models --rows _rows.csv --fit
"""

from __future__ import annotations

import argparse
import csv
import json
import statistics
from pathlib import Path
from typing import Dict, Iterable, List, Optional, Tuple

import torch

from ..cuda.driver import get_device_attributes
from .conv2d_gw8_kernel import conv2d_gw8_kernel_factory
from .conv2d_gw8_params import Conv2dGw8Params
from .conv2d_gw8_wgrad_kernel import conv2d_gw8_wgrad_kernel_factory
from .kernel import device_status
from .performance_model_cache import MODEL_DIR, PerformanceModelCache, params_features

KERNELS = {
    "spio_conv2d_gw8_fprop": (conv2d_gw8_kernel_factory, {}),
    "spio_conv2d_gw8_dgrad": (conv2d_gw8_kernel_factory, {"igrad": True}),
    "spio_conv2d_gw8_wgrad": (conv2d_gw8_wgrad_kernel_factory, {}),
}


def make_args(kernel_name: str, params: Conv2dGw8Params, device) -> tuple:
    """Operands in the order the kernel takes them (random contents, channels_last)."""
    cl = torch.channels_last
    x = torch.randn(params.input_shape, device=device).half().contiguous(memory_format=cl)
    dy = torch.randn(params.output_shape, device=device).half().contiguous(memory_format=cl)
    w = torch.randn(params.weight_shape, device=device).half().contiguous(memory_format=cl)
    if kernel_name.endswith("fprop"):
        bias = torch.randn(params.k, device=device) if params.has_bias else None
        return (torch.empty_like(dy), x, w, bias)
    if kernel_name.endswith("dgrad"):
        return (torch.empty_like(x), dy, w, None)
    dw = torch.empty(params.weight_shape, device=device, dtype=torch.float32).contiguous(memory_format=cl)
    return (dw, x, dy)


def time_kernel(kernel, args, reps: int = 7, flush: Optional[torch.Tensor] = None) -> float:
    """Median milliseconds of one launch; ``flush`` (a buffer larger than L2) is rewritten
    before every timed launch when the operands themselves do not exceed the cache."""
    for _ in range(2):
        kernel(*args)
    times = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        kernel(*args)
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop))
    return statistics.median(times)


def tune(kernel_name: str, params: Conv2dGw8Params, device="cuda", max_configs: int = 0,
         reps: int = 7) -> List[Tuple[float, object]]:
    """(milliseconds, config) for every configuration, fastest first."""
    factory, kwargs = KERNELS[kernel_name]
    device = torch.device(device)
    ordinal = device.index if device.index is not None else torch.cuda.current_device()
    attr = get_device_attributes(ordinal)
    configs = list(factory.configs(params, attr, **kwargs))
    if max_configs and len(configs) > max_configs:
        step = len(configs) / max_configs
        configs = [configs[int(i * step)] for i in range(max_configs)]
    args = make_args(kernel_name, params, device)
    nbytes = sum(a.numel() * a.element_size() for a in args if a is not None)
    flush = None
    if nbytes < 2 * attr.l2_cache_size:
        flush = torch.empty(2 * max(attr.l2_cache_size, 64 << 20), dtype=torch.uint8, device=device)
    rows = []
    for cfg in configs:
        kernel = factory.make_kernel(params, cfg, attr, **kwargs)
        kernel.compile(attr)
        kernel.load(ordinal)
        rows.append((time_kernel(kernel, args, reps=reps, flush=flush), cfg))
    if device_status() != 0:
        raise RuntimeError("a kernel reported a wait time-out while tuning")
    rows.sort(key=lambda r: r[0])
    return rows


def feature_row(kernel_name: str, params, cfg, ms: float) -> Dict[str, float]:
    factory, _ = KERNELS[kernel_name]
    row = params_features(params, factory.per_model_skip_params)
    row.update({k: float(v) for k, v in cfg.as_tune().items()})
    row["ms"] = ms
    return row


def fit_models(rows_by_kernel: Dict[str, List[Dict[str, float]]], out_dir: Path) -> None:
    """One gradient-boosted-tree model per kernel, predicting log-latency."""
    import math

    from .gbt_model import GbtModel

    for name, rows in rows_by_kernel.items():
        if len(rows) < 20:
            continue
        feats = [{k: v for k, v in r.items() if k != "ms"} for r in rows]
        target = [math.log(r["ms"]) for r in rows]
        model = GbtModel.fit(feats, target, n_trees=120, depth=4, learning_rate=0.15, min_leaf=2)
        (out_dir / f"model__{name}__sm_100a.json").write_text(json.dumps(model.to_json()) + "\n")


def parse_shape(text: str) -> Conv2dGw8Params:
    """``n,c,h,w[,r,s,pad[,bias]]``."""
    v = [int(t) for t in text.split(",")]
    n, c, h, w = v[:4]
    r, s = (v[4], v[5]) if len(v) >= 6 else (3, 3)
    pad = v[6] if len(v) >= 7 else r // 2
    return Conv2dGw8Params(n=n, c=c, h=h, w=w, r=r, s=s, padding=pad, has_bias=len(v) >= 8 and bool(v[7]))


def main(argv: Optional[Iterable[str]] = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shape", action="append", required=True, help="n,c,h,w[,r,s,pad[,bias]]")
    ap.add_argument("--kernel", action="append", choices=sorted(KERNELS), help="default: all three")
    ap.add_argument("--out", default=str(MODEL_DIR), help="directory of the tuning tables / models")
    ap.add_argument("--rows", default=None, help="append every measurement to this CSV")
    ap.add_argument("--max-configs", type=int, default=0)
    ap.add_argument("--fit", action="store_true", help="train the per-kernel models from the rows")
    args = ap.parse_args(list(argv) if argv is not None else None)

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    cache = PerformanceModelCache()
    rows_by_kernel: Dict[str, List[Dict[str, float]]] = {}
    for text in args.shape:
        params = parse_shape(text)
        for name in args.kernel or sorted(KERNELS):
            ranked = tune(name, params, max_configs=args.max_configs)
            best_ms, best_cfg = ranked[0]
            cache.record(name, "sm_100a", params, best_cfg, directory=out_dir)
            rows_by_kernel.setdefault(name, []).extend(feature_row(name, params, c, ms) for ms, c in ranked)
            print(f"{name} {params.encode()}: best {best_ms * 1e3:.1f} us {best_cfg} "
                  f"(worst {ranked[-1][0] * 1e3:.1f} us, {len(ranked)} configs)", flush=True)
    if args.rows:
        path = Path(args.rows)
        all_rows = [dict(r, kernel=name) for name, rows in rows_by_kernel.items() for r in rows]
        fields = ["kernel"] + sorted({k for r in all_rows for k in r if k != "kernel"})
        new_file = not path.exists()
        with path.open("a", newline="") as fh:
            wr = csv.DictWriter(fh, fieldnames=fields, restval=0)
            if new_file:
                wr.writeheader()
            wr.writerows(all_rows)
    if args.fit:
        fit_models(rows_by_kernel, out_dir)


if __name__ == "__main__":
    main()
