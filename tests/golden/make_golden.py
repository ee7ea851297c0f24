"""Generates the golden fixtures in this directory FROM THE REFERENCE's own Python code.

Run once, in a container where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

What is imported from the reference (by file path, so its CUDA-only package __init__ is
not executed): ``spio/kernels/conv2d_gw8_params.py`` (shape arithmetic, kernel-name
encoding), ``spio/kernels/stats.py`` + ``conv2d_stats.py`` (byte / MAC counts).  The
expected tensors come from ``torch.nn.functional.conv2d`` on fp32 copies of the fp16
operands with the keyword arguments the reference derives from its Params
(spio/reflection/conv2d_gw8_reflection.py ``_torch_conv2d_kwargs``) and from
``torch.autograd.grad`` of it -- the oracle the reference's tests use for these kernels
(spio/src_tests/run_test.py:43-50, 84-102).  Operands follow the reference's test
distribution, randn clipped to +-3 (spio/reflection/arg_info.py:81-85).

Outputs: ``gw8_cases.npz`` (operands and expected results of small cases),
``gw8_params_stats.json`` (derived shapes, encoded names and statistics) and
``model_shapes.json``: the layer shapes of real models the reference keeps for its tests and
its performance models (spio/src_tests/Conv2dGw8Params.dat, one ``Conv2dGw8Params(...)`` per
line), each evaluated with the reference's own class and stored as plain fields plus the
encoded name.  The tests and the autotuner read only these files; they never read the
reference checkout.
"""

from __future__ import annotations

import importlib.util
import json
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent

# (n, c, h, w, padding, r, s, has_bias): small versions of the shapes the reference tests
# (tests/test_conv2d_gw8.py:67-180): every filter size class, zero / large / asymmetric
# padding, odd extents, one to several groups, channel counts that are not a multiple of 64.
CASES = [
    (2, 16, 6, 5, 1, 3, 3, True),
    (1, 8, 8, 16, 1, 3, 3, False),
    (2, 24, 7, 7, (2, 2), 5, 5, True),
    (2, 16, 9, 9, (2, 0), 4, 1, True),
    (1, 16, 10, 9, 0, 3, 3, False),
    (1, 8, 5, 6, 7, 3, 3, False),
    (3, 72, 4, 4, (0, 1), 1, 2, True),
    (1, 16, 6, 6, (1, 2), 2, 5, False),
]

STATS_SHAPES = [
    dict(n=16, c=128, h=32, w=64, r=3, s=3, padding=1, has_bias=False),
    dict(n=128, c=64, h=56, w=56, r=3, s=3, padding=1, has_bias=False),
    dict(n=256, c=768, h=7, w=7, r=3, s=3, padding=1, has_bias=True),
    dict(n=8, c=64, h=32, w=32, r=3, s=3, padding=1, has_bias=False),
    dict(n=4, c=128, h=20, w=19, r=5, s=4, padding=(2, 0), has_bias=True),
]


def load_reference(root: Path):
    """Import the three pure-Python reference modules under a private package name."""
    pkg = types.ModuleType("_refspio")
    pkg.__path__ = []
    kernels = types.ModuleType("_refspio.kernels")
    kernels.__path__ = [str(root / "spio" / "kernels")]
    sys.modules["_refspio"] = pkg
    sys.modules["_refspio.kernels"] = kernels
    mods = {}
    for name in ("params", "conv2d_gw8_params", "stats", "conv2d_stats"):
        spec = importlib.util.spec_from_file_location(
            f"_refspio.kernels.{name}", root / "spio" / "kernels" / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = mod
        spec.loader.exec_module(mod)
        mods[name] = mod
    return mods["conv2d_gw8_params"].Conv2dGw8Params, mods["conv2d_stats"].Conv2dStats


def randn_clip_3(shape, gen, dtype):
    return torch.clip(torch.randn(shape, generator=gen), -3, 3).to(dtype)


def main(root: Path) -> None:
    Params, Stats = load_reference(root)
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    arrays = {}
    meta = []
    for i, (n, c, h, w, padding, r, s, has_bias) in enumerate(CASES):
        params = Params(n=n, c=c, h=h, w=w, padding=padding, r=r, s=s, has_bias=has_bias)
        params.validate()
        gen = torch.Generator().manual_seed(1000 + i)
        x = randn_clip_3(params.input_shape, gen, torch.float16)
        wt = randn_clip_3(params.weight_shape, gen, torch.float16)
        b = randn_clip_3(params.bias_shape, gen, torch.float32) if has_bias else None
        dy = randn_clip_3(params.output_shape, gen, torch.float16)
        kwargs = {"stride": params.stride, "padding": params.padding, "groups": params.groups}
        xf = x.float().requires_grad_(True)
        wf = wt.float().requires_grad_(True)
        y = torch.nn.functional.conv2d(xf, wf, b, **kwargs)
        dx, dw = torch.autograd.grad(y, (xf, wf), dy.float())
        arrays[f"c{i}_x"] = x.numpy()
        arrays[f"c{i}_w"] = wt.numpy()
        if has_bias:
            arrays[f"c{i}_bias"] = b.numpy()
        arrays[f"c{i}_dy"] = dy.numpy()
        arrays[f"c{i}_y"] = y.detach().numpy()
        arrays[f"c{i}_dx"] = dx.numpy()
        arrays[f"c{i}_dw"] = dw.numpy()
        meta.append(dict(n=n, c=c, h=h, w=w, r=r, s=s, pad_h=params.padding_h,
                         pad_w=params.padding_w, has_bias=has_bias, p=params.p, q=params.q,
                         encode=params.encode()))
    arrays["meta"] = np.frombuffer(json.dumps(meta).encode(), dtype=np.uint8)
    np.savez_compressed(HERE / "gw8_cases.npz", **arrays)

    stats = []
    for kw in STATS_SHAPES:
        params = Params(**kw)
        row = dict(params=dict(kw, padding=list(kw["padding"]) if isinstance(kw["padding"], tuple)
                               else kw["padding"]),
                   encode=params.encode(), groups=params.groups, p=params.p, q=params.q,
                   transpose_padding=[params.transpose_padding_h, params.transpose_padding_w],
                   input_shape=list(params.input_shape), output_shape=list(params.output_shape),
                   weight_shape=list(params.weight_shape), bias_shape=list(params.bias_shape))
        for out in ("output", "grad_input", "grad_weight", "grad_bias"):
            st = Stats(params, output_names=out)
            row[out] = dict(macs=st.macs, bytes_read=st.bytes_read, bytes_written=st.bytes_written,
                            bytes=st.bytes, accumulation_depths=st.accumulation_depths)
        stats.append(row)
    (HERE / "gw8_params_stats.json").write_text(json.dumps(stats, indent=1) + "\n")

    shapes = []
    for line in (root / "spio" / "src_tests" / "Conv2dGw8Params.dat").read_text().splitlines():
        if not line.strip():
            continue
        params = eval(line, {"__builtins__": {}, "Conv2dGw8Params": Params})  # noqa: S307 - the reference's fixture
        params.validate()
        shapes.append(dict(n=params.n, c=params.c, h=params.h, w=params.w, r=params.r, s=params.s,
                           pad_h=params.padding_h, pad_w=params.padding_w, has_bias=bool(params.has_bias),
                           encode=params.encode()))
    (HERE / "model_shapes.json").write_text(json.dumps(shapes, indent=0) + "\n")
    print("wrote", len(shapes), "model shapes")
    print("wrote", HERE / "gw8_cases.npz", (HERE / "gw8_cases.npz").stat().st_size, "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of the andravin/spio checkout>")
    main(Path(sys.argv[1]))
