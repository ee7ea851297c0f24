"""Launch one gw8 kernel a few times on one layer shape through the C ABI -- the smallest program
that exercises a kernel, meant as the target of a profiler capture:

    python -m spio_b200.examples.run_layer fprop 256 128 56 --launches 3
    ncu --set full --clock-control none -k regex:conv2d_gw8_fwd -s 1 -c 2 -o fwd \\
        python -m spio_b200.examples.run_layer fprop 256 128 56 --launches 3

Operands are seeded N(0,1) fp16 NHWC tensors (three sets, used in turn, so that a launch does not
find its operands in the L2 cache); the filter is 3x3, stride 1, padding 1 unless --filter is given.
"""

from __future__ import annotations

import argparse
import ctypes

import torch

from spio_b200 import _clib


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("kind", choices=["fprop", "dgrad", "wgrad", "backward", "layernorm"],
                    help="backward = the combined call (wgrad, reduce, dgrad); "
                         "layernorm = forward + backward of spio::layernorm_2d on an n x c x hw x hw tensor")
    ap.add_argument("n", type=int)
    ap.add_argument("c", type=int)
    ap.add_argument("hw", type=int)
    ap.add_argument("--filter", type=int, default=3, help="filter height and width (padding = filter // 2)")
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--tune", default="", help='JSON tile configuration, e.g. \'{"pps": 1}\'')
    args = ap.parse_args()

    import json

    lib = _clib.load()
    dev = torch.device("cuda:0")
    cl = torch.channels_last
    n, c, hw, r = args.n, args.c, args.hw, args.filter
    if args.kind == "layernorm":
        from spio_b200.functional import layernorm_2d_backward_op, layernorm_2d_op

        gen = torch.Generator(device=dev).manual_seed(1234)
        weight, bias = torch.randn(c, device=dev, generator=gen), torch.randn(c, device=dev, generator=gen)
        xs = [torch.randn(n, c, hw, hw, device=dev, generator=gen).half().contiguous(memory_format=cl) for _ in range(3)]
        for i in range(args.launches):
            y, stats = layernorm_2d_op(xs[i % 3], weight, bias, 1e-6)
            layernorm_2d_backward_op(xs[(i + 1) % 3], xs[i % 3], stats, weight, True, True)
        torch.cuda.synchronize()
        print(f"layernorm {n}x{c}x{hw}x{hw}: {args.launches} forward + backward launches ok")
        return
    sh = _clib.Shape(n, c, hw, hw, r, r, r // 2, r // 2)
    shp = ctypes.byref(sh)
    tune = _clib.make_tune(json.loads(args.tune)) if args.tune else None
    tp = ctypes.byref(tune) if tune is not None else None
    gen = torch.Generator(device=dev).manual_seed(1234)
    sets = 3
    xs = [torch.randn(n, c, hw, hw, device=dev, generator=gen).half().contiguous(memory_format=cl) for _ in range(sets)]
    ys = [torch.randn(n, c, hw, hw, device=dev, generator=gen).half().contiguous(memory_format=cl) for _ in range(sets)]
    w = torch.randn(c, 8, r, r, device=dev, generator=gen).half().contiguous(memory_format=cl)
    dw = torch.empty(c, 8, r, r, device=dev, dtype=torch.float32).contiguous(memory_format=cl)
    dxs = [torch.empty_like(xs[0]) for _ in range(sets)] if args.kind == "backward" else []
    nbytes = lib.spio_conv2d_gw8_wgrad_scratch_bytes(shp, tp if args.kind == "wgrad" else None)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for i in range(args.launches):
        x, y = xs[i % sets], ys[i % sets]
        if args.kind == "fprop":
            rc = lib.spio_conv2d_gw8_fprop(y.data_ptr(), x.data_ptr(), w.data_ptr(), None, shp, tp, stream)
        elif args.kind == "dgrad":
            rc = lib.spio_conv2d_gw8_dgrad(y.data_ptr(), x.data_ptr(), w.data_ptr(), shp, tp, stream)
        elif args.kind == "backward":
            rc = lib.spio_conv2d_gw8_backward(dxs[i % sets].data_ptr(), dw.data_ptr(), None, x.data_ptr(), y.data_ptr(),
                                              w.data_ptr(), shp, None, None, scratch.data_ptr(), nbytes, stream, None)
        else:
            rc = lib.spio_conv2d_gw8_wgrad(dw.data_ptr(), x.data_ptr(), y.data_ptr(), shp, tp, scratch.data_ptr(),
                                           nbytes, stream)
        _clib.check(rc)
    torch.cuda.synchronize()
    if _clib.device_status() != 0:
        raise SystemExit("a kernel reported a wait time-out")
    print(f"{args.kind} {n}x{c}x{hw}x{hw} {r}x{r}: {args.launches} launches ok")


if __name__ == "__main__":
    main()
