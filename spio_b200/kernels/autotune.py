"""Measure tile configurations on the device, keep the best per layer shape, train the model.

The reference collects (kernel, params, config, latency) rows by running a model under
torch.profiler with random configuration overlays and trains one XGBoost regressor per kernel
from them (scripts/profile_block.py:551-701, scripts/train_performance_model.py:46-142).  Here
each configuration of a kernel family's configuration space is timed directly with CUDA events,
in chains of back-to-back launches that rotate over operand sets larger than the L2 cache (the
way the kernels run in a training step; input-gradient and weight-gradient configurations inside
the combined backward call, whose time is what their rows hold); the fastest goes into the tuning table that
``PerformanceModelCache`` consults first, and all rows can be fitted by the small
gradient-boosted-tree model in ``gbt_model.py`` for shapes that were never measured.

    python -m spio_b200.kernels.autotune --shape 256,64,56,56 --shapes-file tests/golden/model_shapes.json \
        --out spio_b200/kernels/perf_models --rows rows.csv          # on the GPU
    python -m spio_b200.kernels.autotune --from-rows rows.csv --out spio_b200/kernels/perf_models   # anywhere
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
from .kernel import device_status, launch_backward
from .performance_model_cache import MODEL_DIR, PerformanceModelCache, params_features

KERNELS = {
    "spio_conv2d_gw8_fprop": (conv2d_gw8_kernel_factory, {}),
    "spio_conv2d_gw8_dgrad": (conv2d_gw8_kernel_factory, {"igrad": True}),
    "spio_conv2d_gw8_wgrad": (conv2d_gw8_wgrad_kernel_factory, {}),
}


def make_operand_sets(kernel_name: str, params: Conv2dGw8Params, device, min_bytes: int) -> List[tuple]:
    """Operand sets in the order the kernel takes them (random contents, channels_last), as many
    as it takes for the streamed tensors to total ``min_bytes``: a timed chain rotates over them,
    so no launch finds its operands in the L2 cache.  Weights and bias are shared."""
    cl = torch.channels_last
    w = torch.randn(params.weight_shape, device=device).half().contiguous(memory_format=cl)
    bias = torch.randn(params.k, device=device) if params.has_bias else None
    per_set = 2 * (params.n * params.c * params.h * params.w + params.n * params.k * params.p * params.q)
    sets = max(2, -(-min_bytes // per_set))
    out = []
    for _ in range(sets):
        x = torch.randn(params.input_shape, device=device).half().contiguous(memory_format=cl)
        dy = torch.randn(params.output_shape, device=device).half().contiguous(memory_format=cl)
        if kernel_name.endswith("fprop"):
            out.append((torch.empty_like(dy), x, w, bias))
        elif kernel_name.endswith("dgrad"):
            out.append((torch.empty_like(x), dy, w, None))
        else:
            dw = torch.empty(params.weight_shape, device=device, dtype=torch.float32).contiguous(memory_format=cl)
            out.append((dw, x, dy))
    return out


def make_backward_sets(params: Conv2dGw8Params, device, min_bytes: int) -> List[tuple]:
    """Operand sets of the combined backward call, (dx, dw, x, dy, w, dbias): the input-gradient and
    the weight-gradient configurations are timed inside that call, next to the other kernel with
    the planner's defaults, because that is where they run: a configuration that wins a chain of
    identical launches can lose there (a deeper ring that changes the SM's shared-memory
    configuration cost the backward call of 256 x 256 x 28 x 28 11 us)."""
    cl = torch.channels_last
    w = torch.randn(params.weight_shape, device=device).half().contiguous(memory_format=cl)
    dw = torch.empty(params.weight_shape, device=device, dtype=torch.float32).contiguous(memory_format=cl)
    fused_bias = params.has_bias and (params.r * params.s) % 2 == 1
    dbias = torch.empty(params.k, device=device, dtype=torch.float32) if fused_bias else None
    per_set = 2 * (2 * params.n * params.c * params.h * params.w + params.n * params.k * params.p * params.q)
    sets = max(2, -(-min_bytes // per_set))
    out = []
    for _ in range(sets):
        x = torch.randn(params.input_shape, device=device).half().contiguous(memory_format=cl)
        dy = torch.randn(params.output_shape, device=device).half().contiguous(memory_format=cl)
        out.append((torch.empty_like(x), dw, x, dy, w, dbias))
    return out


def time_kernel(kernel, operand_sets: List[tuple], reps: int = 3, target_ms: float = 1.0) -> float:
    """Median milliseconds per launch in chains of back-to-back launches over rotating operand
    sets: the way the kernels run in a training step (programmatic dependent launch lets a
    launch's prologue overlap its predecessor's tail), with a cold L2 for every launch."""
    k = len(operand_sets)
    for i in range(2):
        kernel(*operand_sets[i % k])
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    kernel(*operand_sets[0])
    stop.record()
    stop.synchronize()
    count = max(4, min(24, int(target_ms / max(start.elapsed_time(stop), 1e-3))))
    times = []
    for _ in range(reps):
        # a spin kernel holds the stream for about a millisecond while the host queues the chain, so
        # that the figure is device time even where a call costs the host more than the GPU
        torch.cuda._sleep(2_000_000)
        start.record()
        for i in range(count):
            kernel(*operand_sets[i % k])
        stop.record()
        stop.synchronize()
        times.append(start.elapsed_time(stop) / count)
    return statistics.median(times)


def tune(kernel_name: str, params: Conv2dGw8Params, device="cuda", max_configs: int = 0,
         reps: int = 3) -> List[Tuple[float, object]]:
    """(milliseconds, config) for every configuration, fastest first."""
    factory, kwargs = KERNELS[kernel_name]
    device = torch.device(device)
    ordinal = device.index if device.index is not None else torch.cuda.current_device()
    attr = get_device_attributes(ordinal)
    configs = list(factory.configs(params, attr, **kwargs))
    if max_configs and len(configs) > max_configs:
        step = len(configs) / max_configs
        configs = [configs[int(i * step)] for i in range(max_configs)]
    # the launch planner's own choice (every field open) is always a candidate: it is what a table
    # entry has to beat
    default = type(configs[0])() if configs else None
    if default is not None and default not in configs:
        configs.insert(0, default)
    backward = not kernel_name.endswith("fprop")
    sets = (make_backward_sets(params, device, min_bytes=4 * attr.l2_cache_size) if backward
            else make_operand_sets(kernel_name, params, device, min_bytes=4 * attr.l2_cache_size))
    partner = None
    if backward:
        # the other kernel of the backward call, with the planner's defaults
        other, other_kwargs = KERNELS["spio_conv2d_gw8_wgrad" if kernel_name.endswith("dgrad") else "spio_conv2d_gw8_dgrad"]
        partner = other.make_kernel(params, None, attr, **other_kwargs)
        partner.compile(attr)
        partner.load(ordinal)
    rows = []
    for cfg in configs:
        kernel = factory.make_kernel(params, cfg, attr, **kwargs)
        kernel.compile(attr)
        kernel.load(ordinal)
        if backward:
            wk, dk = (partner, kernel) if kernel_name.endswith("dgrad") else (kernel, partner)
            call = lambda dx, dw, x, dy, w, db, wk=wk, dk=dk: launch_backward(wk, dk, dx, dw, x, dy, w, db)  # noqa: E731
        else:
            call = kernel
        rows.append((time_kernel(call, sets, reps=reps), cfg))
    if device_status() != 0:
        raise RuntimeError("a kernel reported a wait time-out while tuning")
    rows.sort(key=lambda r: r[0])
    return rows


# A configuration enters the tuning table only if it beats the launch planner's defaults by this
# margin: smaller differences are within what two timings of one configuration differ by, and a
# choice made on a chain of identical launches need not hold inside a training step, where the
# kernels alternate.
TABLE_MARGIN = 0.97


def pick(ranked: List[Tuple[float, object]]) -> Tuple[float, object]:
    """The table entry for a shape: the fastest configuration, or the planner's defaults (a
    configuration with every field open) unless the fastest one is faster by TABLE_MARGIN."""
    best_ms, best_cfg = ranked[0]
    for ms, cfg in ranked:
        if not any(cfg.as_tune().values()):
            if best_ms > TABLE_MARGIN * ms:
                return ms, cfg
            break
    return best_ms, best_cfg


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


def read_rows(path: Path) -> Dict[str, List[Dict[str, float]]]:
    """Timing rows written by ``--rows``, grouped by kernel."""
    out: Dict[str, List[Dict[str, float]]] = {}
    with Path(path).open(newline="") as fh:
        for row in csv.DictReader(fh):
            name = row.pop("kernel")
            out.setdefault(name, []).append({k: float(v) for k, v in row.items()})
    return out


def shapes_from_file(path: Path, max_batch: int = 0) -> List[Conv2dGw8Params]:
    """Layer shapes from a JSON list of {n, c, h, w, r, s, pad_h, pad_w, has_bias} records (the
    format of tests/golden/model_shapes.json)."""
    out = []
    for d in json.loads(Path(path).read_text()):
        n = min(d["n"], max_batch) if max_batch else d["n"]
        out.append(Conv2dGw8Params(n=n, c=d["c"], h=d["h"], w=d["w"], r=d["r"], s=d["s"],
                                   padding=(d["pad_h"], d["pad_w"]), has_bias=bool(d["has_bias"])))
    return out


def parse_shape(text: str) -> Conv2dGw8Params:
    """``n,c,h,w[,r,s,pad[,bias]]``."""
    v = [int(t) for t in text.split(",")]
    n, c, h, w = v[:4]
    r, s = (v[4], v[5]) if len(v) >= 6 else (3, 3)
    pad = v[6] if len(v) >= 7 else r // 2
    return Conv2dGw8Params(n=n, c=c, h=h, w=w, r=r, s=s, padding=pad, has_bias=len(v) >= 8 and bool(v[7]))


def main(argv: Optional[Iterable[str]] = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--shape", action="append", default=[], help="n,c,h,w[,r,s,pad[,bias]]")
    ap.add_argument("--shapes-file", default=None, help="JSON list of layer shapes (tests/golden/model_shapes.json)")
    ap.add_argument("--from-rows", default=None,
                    help="fit the models from a CSV written by --rows (no GPU needed) and exit")
    ap.add_argument("--kernel", action="append", choices=sorted(KERNELS), help="default: all three")
    ap.add_argument("--out", default=str(MODEL_DIR), help="directory of the tuning tables / models")
    ap.add_argument("--rows", default=None, help="append every measurement to this CSV")
    ap.add_argument("--max-configs", type=int, default=0)
    ap.add_argument("--fit", action="store_true", help="train the per-kernel models from the rows")
    args = ap.parse_args(list(argv) if argv is not None else None)

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    if args.from_rows:
        fit_models(read_rows(Path(args.from_rows)), out_dir)
        return
    cache = PerformanceModelCache()
    rows_by_kernel: Dict[str, List[Dict[str, float]]] = {}
    shapes = [parse_shape(text) for text in args.shape]
    if args.shapes_file:
        shapes += shapes_from_file(Path(args.shapes_file))
    if not shapes:
        ap.error("give --shape and / or --shapes-file")
    seen = set()
    for params in shapes:
        if params.encode() in seen:
            continue
        seen.add(params.encode())
        for name in args.kernel or sorted(KERNELS):
            ranked = tune(name, params, max_configs=args.max_configs)
            best_ms, best_cfg = pick(ranked)
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
