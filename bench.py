"""Benchmark of the gw8 convolution training step (fprop + wgrad + dgrad) on B200.

    python bench.py --gpus N --steps K --warmup W            # this package's CUDA kernels
    python bench.py --impl reference --gpus N ...            # CPU baseline arm

Workload (default): the data-parallel sweep layer -- C=K=64, 56x56, 3x3, stride 1, pad 1,
group width 8, fp16 NHWC -- with a GLOBAL batch of 2048 images sharded over the N ranks
(strong scaling).  One step = forward, weight gradient, input gradient on the rank's
shard; with N > 1 the fp32 weight gradient is summed over the ranks inside the step's chain
of dependent launches (peer stores over NVLink + a rank-order sum; an NCCL all-reduce on a
side stream if the exchange buffers cannot be set up).  Synthetic seeded N(0,1) activations /
gradients and N(0, 1/sqrt(72)) weights.  Every operand streamed by a kernel is larger than the
126 MB L2 at every N (>= 205 MB per kernel launch at N=8), so no L2 flush is needed between
steps.

Prints ONE JSON line (rank 0).  ``value`` is whole-job effective bandwidth: algorithmic
bytes of the three kernels over all ranks (spio_b200.kernels.Conv2dStats, 2 bytes per
element, each operand once) divided by the device time of a step, max over ranks.

Extra keys of the line (single-GPU run): ``sustained`` (>= 200 steps with the sampled clocks),
``sweep`` (the batch sweep of the 64-channel 56x56 layer at N = 128, 256, 512: per kernel through
the C ABI with the planner's defaults, and through the PyTorch operator, which takes its tile
configurations from the tuning tables), ``ladder`` (the channel / resolution ladder at N = 256),
``convnext_step_ms`` (the ConvNeXt-T-style train step at batch 256, and the same network as stock
torch runs it) and ``host_us_per_call``.  Each sweep / ladder point also carries the incumbents
on the same operands: the reference's own kernels (when oracle/_ref was built) and torch's
grouped convolution through cuDNN.
Kernels of the sweep and the ladder are timed in chains of back-to-back launches that rotate
over operand sets totalling more than 600 MB, so every launch finds a cold L2.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GLOBAL_BATCH = 2048
C, H, W, R, S, PAD = 64, 56, 56, 3, 3, 1
ROTATE_BYTES = 600 << 20  # operand sets a timed chain rotates over (> 4 x the 126 MB L2)
# DRAM traffic of one forward-kernel launch, from an ncu capture at N=512: reads are 1.015 x the
# input bytes (halo rows at span ends); writes are the output bytes minus ~48 MB that are still
# dirty in the 126 MB L2 when the kernel ends.  Reads and writes grow with the batch, the L2
# residue does not, so a launch at another batch is estimated as below.
FWD_DRAM_READ_RATIO = 1.015
FWD_L2_RESIDUE_BYTES = 47.7e6
CL = torch.channels_last


def fwd_dram_traffic(algorithmic: int) -> float:
    half = algorithmic / 2.0
    return FWD_DRAM_READ_RATIO * half + max(half - FWD_L2_RESIDUE_BYTES, 0.0)


def algorithmic_bytes(n: int, c: int = C, hw: int = H) -> int:
    """Bytes of ONE of the three kernels for a batch of n (identical for all three)."""
    from spio_b200.kernels import Conv2dGw8Params, Conv2dStats

    return Conv2dStats(Conv2dGw8Params(n=n, c=c, h=hw, w=hw, padding=PAD, r=R, s=S),
                       output_names="output").bytes


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """SM clock, power and throttle reasons of one GPU, read (never set) through NVML on a
    thread every few milliseconds while the timed region runs."""

    REASONS = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "hw_thermal_slowdown": 0x40,
               "sw_thermal_slowdown": 0x20}

    def __init__(self, index: int, period_s: float = 0.002):
        self.index = index
        self.period_s = period_s
        self.rows = []
        self.thread = None
        self.stop_flag = threading.Event()
        self.error = None
        self.handle = None
        self.nvml = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except TypeError:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self.nvml = pynvml
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception as exc:  # no NVML: report it instead of numbers
            self.error = f"NVML unavailable: {exc}"
            return
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _run(self):
        nv, h = self.nvml, self.handle
        while not self.stop_flag.is_set():
            try:
                self.rows.append((nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM),
                                  nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
                                  nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                                  if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons")
                                  else nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)))
            except Exception as exc:
                self.error = f"NVML read failed: {exc}"
                return
            time.sleep(self.period_s)

    def stop(self) -> dict:
        if self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.error or "not started"]}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [self.error or "no samples"]}
        bits = 0
        for r in self.rows:
            bits |= int(r[2])
        return {"sm_mhz": statistics.median(r[0] for r in self.rows), "sm_max_mhz": self.sm_max,
                "sm_mhz_min": min(r[0] for r in self.rows),
                "power_w_max": max(r[1] for r in self.rows), "samples": len(self.rows),
                "reasons": sorted(name for name, bit in self.REASONS.items() if bits & bit)}


# ------------------------------------------------------------------------------ timing helpers

def chain_us(launch, count: int, reps: int = 5, hold_ms: float = 0.0) -> float:
    """Median microseconds per launch of ``count`` back-to-back ``launch(i)`` calls, timed with
    CUDA events on the current stream.  With ``hold_ms`` a spin kernel occupies the stream
    first, so that the host has queued the whole chain before the GPU starts it and the figure
    is device time even when one call costs the host more than it costs the GPU."""
    stream = torch.cuda.current_stream()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        if hold_ms > 0:
            torch.cuda._sleep(int(hold_ms * 1.9e6))
        e0.record(stream)
        for i in range(count):
            launch(i)
        e1.record(stream)
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / count)
    return statistics.median(times)


def host_us(launch, count: int) -> float:
    """Host microseconds per un-synchronised call."""
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for i in range(count):
        launch(i)
    dt = time.perf_counter() - t0
    torch.cuda.synchronize()
    return dt / count * 1e6


class LayerPoint:
    """One layer shape at one batch size: operand sets to rotate over and the timed chains."""

    def __init__(self, lib, dev, n: int, c: int, hw: int, seed: int):
        from spio_b200 import _clib

        self.lib, self.dev, self.n, self.c, self.hw = lib, dev, n, c, hw
        self.clib = _clib
        self.sh = _clib.Shape(n, c, hw, hw, R, S, PAD, PAD)
        self.shp = ctypes.byref(self.sh)
        per_set = 2 * n * c * hw * hw * 2
        self.sets = max(2, ROTATE_BYTES // per_set + 1)
        gen = torch.Generator(device=dev).manual_seed(seed)
        mk = lambda: torch.randn(n, c, hw, hw, device=dev, generator=gen).half().contiguous(memory_format=CL)  # noqa: E731
        self.a = [mk() for _ in range(self.sets)]            # x, or dy
        self.b = [mk() for _ in range(self.sets)]            # dy for the backward kernels, or outputs
        self.out = [torch.empty_like(self.a[0]) for _ in range(self.sets)]
        self.w = (torch.randn(c, 8, R, S, device=dev, generator=gen) / 72 ** 0.5).half().contiguous(memory_format=CL)
        self.dw = torch.empty(c, 8, R, S, device=dev, dtype=torch.float32).contiguous(memory_format=CL)
        self.scratch_bytes = lib.spio_conv2d_gw8_wgrad_scratch_bytes(self.shp, None)
        self.scratch = torch.empty(self.scratch_bytes, dtype=torch.uint8, device=dev)
        self.bytes = algorithmic_bytes(n, c, hw)

    def c_abi(self, count: int = 40) -> dict:
        # The kernels' time follows the SM clock at small batch, and the clock sags for a while after
        # a long stretch of full load: let the board settle, and record the clock seen while timing.
        torch.cuda.synchronize()
        time.sleep(0.3)
        sampler = ClockSampler(self.dev.index or 0, period_s=0.001)
        sampler.start()
        try:
            res = self._c_abi(count)
        finally:
            clocks = sampler.stop()
        res["sm_mhz"] = {k: clocks.get(k) for k in ("sm_mhz", "sm_mhz_min", "samples")}
        return res

    def _c_abi(self, count: int) -> dict:
        lib, shp, chk = self.lib, self.shp, self.clib.check
        sp = torch.cuda.current_stream(self.dev).cuda_stream
        k = self.sets

        def fprop(i):
            chk(lib.spio_conv2d_gw8_fprop(self.out[i % k].data_ptr(), self.a[i % k].data_ptr(), self.w.data_ptr(),
                                          None, shp, None, sp))

        def dgrad(i):
            chk(lib.spio_conv2d_gw8_dgrad(self.out[i % k].data_ptr(), self.b[i % k].data_ptr(), self.w.data_ptr(),
                                          shp, None, sp))

        def wgrad(i):
            chk(lib.spio_conv2d_gw8_wgrad(self.dw.data_ptr(), self.a[i % k].data_ptr(), self.b[i % k].data_ptr(), shp,
                                          None, self.scratch.data_ptr(), self.scratch_bytes, sp))

        def step(i):
            fprop(i)
            chk(lib.spio_conv2d_gw8_backward(self.out[(i + 1) % k].data_ptr(), self.dw.data_ptr(), None,
                                             self.a[i % k].data_ptr(), self.b[i % k].data_ptr(), self.w.data_ptr(),
                                             shp, None, None, self.scratch.data_ptr(), self.scratch_bytes, sp, None))

        res = {}
        for name, fn in (("fprop", fprop), ("dgrad", dgrad), ("wgrad", wgrad)):
            for i in range(count):
                fn(i)
            us = chain_us(fn, count)
            res[name] = self._rate(us)
        # warm variant: every launch works on the same operand set, so whatever part of it fits in the
        # 126 MB L2 is found there (a layer's input is usually what the kernel before it just wrote);
        # the rate may exceed the HBM roofline and is labelled, not compared with it
        res["warm_l2"] = {name: dict(self._rate(chain_us(lambda i, fn=fn: fn(0), count)),
                                     note="same operand set every launch; not an HBM figure")
                          for name, fn in (("fprop", fprop), ("dgrad", dgrad), ("wgrad", wgrad))}
        def backward(i):
            chk(lib.spio_conv2d_gw8_backward(self.out[i % k].data_ptr(), self.dw.data_ptr(), None,
                                             self.a[i % k].data_ptr(), self.b[i % k].data_ptr(), self.w.data_ptr(),
                                             shp, None, None, self.scratch.data_ptr(), self.scratch_bytes, sp, None))

        # wgrad -> reduce -> dgrad as the operator's backward pass issues them: the input-gradient kernel does
        # not wait for the reduction, which costs a chain of bare wgrad + reduce launches about 4 us per launch
        for i in range(8):
            backward(i)
        us = chain_us(backward, count // 2)
        res["backward"] = dict(self._rate(us / 2.0), us=us)
        for i in range(8):
            step(i)
        us = chain_us(step, count // 2)
        res["step"] = dict(self._rate(us / 3.0), us=us)
        res["host_us_per_call"] = {"fprop": host_us(fprop, 200), "wgrad": host_us(wgrad, 200)}
        return res

    def operator(self, count: int = 20) -> dict:
        """The same layer through torch.ops.spio.conv2d_gw8 and autograd, as Conv2dGw8.forward runs it."""
        from spio_b200.functional import conv2d_gw8
        from spio_b200.kernels import (Conv2dGw8Params, conv2d_gw8_kernel_factory,
                                       conv2d_gw8_wgrad_kernel_factory)

        k = self.sets
        xs = [t.detach().requires_grad_(True) for t in self.a]
        w = self.w.detach().requires_grad_(True)
        groups = self.c // 8

        keep = [None] * k   # outputs stay alive, as activations do in a network: the allocator hands out k buffers in turn

        def fwd(i):
            with torch.no_grad():
                keep[i % k] = conv2d_gw8(xs[i % k], w, None, 1, PAD, PAD, 1, groups)

        kept = [None] * k

        def step(i):
            y = conv2d_gw8(xs[i % k], w, None, 1, PAD, PAD, 1, groups)
            # y and the gradients stay alive for k steps: otherwise the allocator hands every step the block
            # the step before it freed, and outputs rewritten in place partly stay in the L2 cache
            kept[i % k] = (y, torch.autograd.grad(y, (xs[i % k], w), self.b[i % k]))

        for i in range(4):
            step(i)
        fwd_us = chain_us(fwd, count, hold_ms=4.0)
        step_us = chain_us(step, count, hold_ms=12.0)
        host_step_us = host_us(step, 50)
        # The same steps, one per operand set, captured into one CUDA graph: what the operator costs the
        # device when the host is out of the way (recorded launches split their work statically).
        graph_us = None
        try:
            # leaf tensors of the captured steps' own, first used on the capturing stream (autograd
            # synchronises every backward pass with the stream a leaf was first used on)
            gxs = [t.detach().requires_grad_(True) for t in self.a]
            gw = self.w.detach().requires_grad_(True)
            gkept = [None] * k

            def gstep(i):
                y = conv2d_gw8(gxs[i % k], gw, None, 1, PAD, PAD, 1, groups)
                gkept[i % k] = (y, torch.autograd.grad(y, (gxs[i % k], gw), self.b[i % k]))

            side = torch.cuda.Stream(self.dev)
            side.wait_stream(torch.cuda.current_stream(self.dev))
            with torch.cuda.stream(side):
                gstep(0)
            torch.cuda.current_stream(self.dev).wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for i in range(k):
                    gstep(i)
            graph.replay()
            graph_us = chain_us(lambda i: graph.replay(), max(2, count // k), reps=3) / k
            del graph
        except Exception as exc:  # a figure less, not a failed run
            graph_us = f"not captured: {str(exc)[:120]}"
        params = Conv2dGw8Params(n=self.n, c=self.c, h=self.hw, w=self.hw, padding=PAD, r=R, s=S)
        chosen = {}
        for name, fac, kw in (("fprop", conv2d_gw8_kernel_factory, {}), ("dgrad", conv2d_gw8_kernel_factory, {"igrad": True}),
                              ("wgrad", conv2d_gw8_wgrad_kernel_factory, {})):
            kern = fac.get_kernel(params, self.dev, **kw)
            chosen[name] = {f: v for f, v in kern.config.as_tune().items() if v} if kern.config is not None else {}
        return {"fprop": self._rate(fwd_us), "step": dict(self._rate(step_us / 3.0), us=step_us),
                "backward_us": step_us - fwd_us, "host_us_per_step": host_step_us,
                "cuda_graph_step_us": graph_us, "configs": chosen}

    def incumbent(self, count: int = 24) -> dict:
        """The REFERENCE's own kernels for this shape (compiled for sm_100a into oracle/_ref by
        oracle/build_ref_kernels.py), timed in the same chains over the same rotating operands; per
        kernel the fastest of the configurations that were built.  They are launched as the reference
        launches them: plain cuLaunchKernel, and a zero fill of grad_weight before every wgrad."""
        from oracle import ref_kernels

        k = self.sets
        res = {}
        for kind in ("fprop", "dgrad", "wgrad"):
            best = None
            for kern in ref_kernels.kernels_for(kind, self.n, self.c, self.hw, self.hw):
                kern.load()
                if kind == "fprop":
                    fn = lambda i, kern=kern: kern(self.out[i % k], self.a[i % k], self.w, None)  # noqa: E731
                elif kind == "dgrad":
                    fn = lambda i, kern=kern: kern(self.out[i % k], self.b[i % k], self.w)  # noqa: E731
                else:
                    def fn(i, kern=kern):
                        self.dw.zero_()
                        kern(self.dw, self.a[i % k], self.b[i % k])
                for i in range(4):
                    fn(i)
                us = chain_us(fn, count, reps=3)
                if best is None or us < best[0]:
                    best = (us, kern.config)
                kern.unload()
            if best is not None:
                res[kind] = dict(self._rate(best[0]), config=best[1])
        if len(res) == 3:
            us = sum(res[kind]["us"] for kind in res)
            res["step"] = dict(self._rate(us / 3.0), us=us)
        return res

    def cudnn(self, count: int = 20) -> dict:
        """torch's own grouped convolution (cuDNN, fp16, channels_last, algorithm search on) on the same
        rotating operands: forward alone, and forward + autograd of input and weight."""
        import torch.nn.functional as F

        k = self.sets
        groups = self.c // 8
        xs = [t.detach().requires_grad_(True) for t in self.a]
        w = self.w.detach().requires_grad_(True)
        keep = [None] * k
        was = torch.backends.cudnn.benchmark
        torch.backends.cudnn.benchmark = True

        def fwd(i):
            with torch.no_grad():
                keep[i % k] = F.conv2d(xs[i % k], w, None, 1, PAD, 1, groups)

        kept = [None] * k

        def step(i):
            y = F.conv2d(xs[i % k], w, None, 1, PAD, 1, groups)
            kept[i % k] = (y, torch.autograd.grad(y, (xs[i % k], w), self.b[i % k]))  # as in operator()

        try:
            for i in range(3):
                fwd(i)
                step(i)
            fwd_us = chain_us(fwd, count, reps=3)
            step_us = chain_us(step, count, reps=3)
        finally:
            torch.backends.cudnn.benchmark = was
        return {"fprop": self._rate(fwd_us), "step": dict(self._rate(step_us / 3.0), us=step_us),
                "backward_us": step_us - fwd_us}

    def _rate(self, us: float) -> dict:
        peak, _ = measured_peak()
        gbs = self.bytes / us / 1e3
        return {"us": us, "GBps": gbs, "frac_of_measured_peak": gbs / peak}


def convnext_step_ms(dev, batch: int = 256, steps: int = 5, stock: bool = False) -> dict:
    """Train step (forward + backward, fp16 autocast) of the ConvNeXt-T-style network with its 18
    gw8 convolutions and 22 channel LayerNorms swapped for this package's layers; with ``stock`` the
    same network as torch builds it (cuDNN grouped convolutions, torch's LayerNorm), for comparison."""
    from spio_b200.examples.convnext_gw8 import ConvNeXtGw8, swap_layernorm, train_step
    from spio_b200.transform._transform import _transform

    torch.manual_seed(1234 + 4)
    model = ConvNeXtGw8().to(dev).to(memory_format=CL)
    images = torch.randn(batch, 3, 224, 224, device=dev).contiguous(memory_format=CL)
    labels = torch.randint(0, 1000, (batch,), device=dev)
    if stock:
        fused, n_conv, n_ln = model, 0, 0
        torch.backends.cudnn.benchmark = True
    else:
        n_ln = swap_layernorm(model)
        fused, n_conv = _transform(model)
    for _ in range(3):
        fused.zero_grad(set_to_none=True)
        train_step(fused, images, labels)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fused.zero_grad(set_to_none=True)
        loss = train_step(fused, images, labels)
    e1.record()
    torch.cuda.synchronize()
    out = {"ms": e0.elapsed_time(e1) / steps, "batch": batch, "gw8_layers": n_conv, "layernorm2d_layers": n_ln,
           "loss": float(loss), "steps": steps}
    del fused, model, images
    torch.cuda.empty_cache()
    return out


def copy_ceiling(dev, world: int, dist, nbytes: int = 256 << 20) -> float:
    """Aggregate GB/s (both directions, all ranks at once) of plain pinned-memory copies: one
    host-to-device and one device-to-host stream per rank, 256 MB each way."""
    up, down = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    h_in = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    h_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    d_in = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    d_out = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    best = float("inf")
    for _ in range(3):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        with torch.cuda.stream(up):
            d_in.copy_(h_in, non_blocking=True)
        with torch.cuda.stream(down):
            h_out.copy_(d_out, non_blocking=True)
        up.synchronize()
        down.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        best = min(best, float(dt.item()))
    return world * 2 * nbytes / best / 1e9


# ------------------------------------------------------------------------------ our arm

def run_ours(args) -> None:
    import torch.distributed as dist

    from spio_b200 import _clib
    from spio_b200.distributed import PeerExchange

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run for --gpus > 1")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    global_batch = args.global_batch
    n = global_batch // world
    lib = _clib.load()
    sh = _clib.Shape(n, C, H, W, R, S, PAD, PAD)
    shp = ctypes.byref(sh)

    gen = torch.Generator(device=dev).manual_seed(1234 + 5 + rank)
    x = torch.randn(n, C, H, W, device=dev, generator=gen).half().contiguous(memory_format=CL)
    dy = torch.randn(n, C, H, W, device=dev, generator=gen).half().contiguous(memory_format=CL)
    wgen = torch.Generator(device=dev).manual_seed(1234 + 5)
    w = (torch.randn(C, 8, R, S, device=dev, generator=wgen) / 72 ** 0.5).half().contiguous(memory_format=CL)
    y = torch.empty_like(x)
    dx = torch.empty_like(x)
    dw = torch.empty(C, 8, R, S, device=dev, dtype=torch.float32).contiguous(memory_format=CL)

    main = torch.cuda.current_stream(dev)
    sp = main.cuda_stream

    # ---- the collective: peer-store exchange inside the launch chain, else NCCL on a side stream
    px, px_all, collective = None, None, "none (1 GPU)"
    if world > 1:
        collective = "nccl all-reduce on a side stream, overlapped with dgrad"
        if args.collective in ("peer", "auto"):
            try:
                px = px_all = PeerExchange(C * 8 * R * S + C, device=dev)
                collective = "peer-store exchange inside the launch chain (spio_dp_push / spio_dp_sum)"
            except Exception as exc:  # IPC not available here: the NCCL route still works
                collective += f" (peer exchange unavailable: {exc})"
        if px is not None:
            # trial run: the exchange must give the bits of a rank-order sum (checked against NCCL's sum
            # of the same vector, which may differ in the last bit) before the timed steps rely on it
            try:
                probe = torch.randn(C * 8 * R * S, device=dev)
                want = probe.clone()
                dist.all_reduce(want)
                for _ in range(3):
                    got = probe.clone()
                    dp = px.options()
                    _clib.check(lib.spio_dp_allreduce(ctypes.byref(dp), got.data_ptr(), got.numel(), None, 0, sp))
                    px.advance()
                    torch.cuda.synchronize(dev)
                    if _clib.device_status() != 0 or not torch.allclose(got, want, rtol=1e-5, atol=1e-5):
                        raise RuntimeError("trial exchange gave a wrong sum or timed out")
            except Exception as exc:
                collective += f" (peer exchange rejected: {exc})"
                px = None   # the buffers stay mapped until the end: peers may still be storing into them
        ok = torch.tensor([1 if px is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 0 and px is not None:   # all ranks must agree on the route
            px = None
            collective = "nccl all-reduce on a side stream, overlapped with dgrad (peer exchange failed on a rank)"
    if world == 1 and args.force_exchange:   # one rank exchanging with itself: the cost of the chain alone
        px = PeerExchange(C * 8 * R * S + C, device=dev)
        collective = "peer-store exchange with itself (1 GPU, --force-exchange)"
    comm = torch.cuda.Stream(dev) if world > 1 and px is None else None

    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    tunes = json.loads(args.tune) if args.tune else {}
    dgrad_cfg = dict(tunes.get("dgrad", {}))
    if comm is not None:
        # the NCCL kernel needs an SM beside the persistent CTAs (one per SM) to overlap dgrad
        dgrad_cfg.setdefault("grid", sms - 1)
    fprop_tune = _clib.make_tune(tunes["fprop"]) if tunes.get("fprop") else None
    wgrad_tune = _clib.make_tune(tunes["wgrad"]) if tunes.get("wgrad") else None
    dgrad_tune = _clib.make_tune(dgrad_cfg) if dgrad_cfg else None
    fprop_tp = ctypes.byref(fprop_tune) if fprop_tune is not None else None
    wgrad_tp = ctypes.byref(wgrad_tune) if wgrad_tune is not None else None
    dgrad_tp = ctypes.byref(dgrad_tune) if dgrad_tune is not None else None
    scratch_bytes = lib.spio_conv2d_gw8_wgrad_scratch_bytes(shp, wgrad_tp)
    scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=dev)
    dw_ready = torch.cuda.Event()
    dw_ready.record(torch.cuda.current_stream(dev))  # creates the underlying CUDA event

    def fprop(xt=x, yt=y, shape=shp):
        _clib.check(lib.spio_conv2d_gw8_fprop(yt.data_ptr(), xt.data_ptr(), w.data_ptr(), None, shape, fprop_tp, sp))

    def wgrad():
        _clib.check(lib.spio_conv2d_gw8_wgrad(dw.data_ptr(), x.data_ptr(), dy.data_ptr(), shp, wgrad_tp,
                                              scratch.data_ptr(), scratch_bytes, sp))

    def dgrad():
        _clib.check(lib.spio_conv2d_gw8_dgrad(dx.data_ptr(), dy.data_ptr(), w.data_ptr(), shp, dgrad_tp, sp))

    def backward(xt=x, dyt=dy, dxt=dx, dwt=dw, shape=shp):
        """wgrad -> reduce -> [push] -> dgrad -> [sum], chained with programmatic dependent launch."""
        dp = px.options() if px is not None else None
        opts = _clib.BackwardOpts(0, None, None, None, ctypes.pointer(dp) if dp is not None else None)
        _clib.check(lib.spio_conv2d_gw8_backward_ex(
            dxt.data_ptr(), dwt.data_ptr(), None, xt.data_ptr(), dyt.data_ptr(), w.data_ptr(), shape, dgrad_tp,
            wgrad_tp, scratch.data_ptr(), scratch_bytes, sp, dw_ready.cuda_event if comm is not None else None,
            ctypes.byref(opts)))
        if px is not None:
            px.advance()

    def reduce_dw(dwt=dw):
        if comm is not None:
            comm.wait_event(dw_ready)
            with torch.cuda.stream(comm):
                dist.all_reduce(dwt)
            main.wait_stream(comm)

    def step(events=None):
        """One training step of the layer.  With `events` the three kernels are launched
        separately so that each can be timed; otherwise backward is one library call."""
        if events is None:
            fprop()
            backward()
            reduce_dw()
            return
        events[0].record(main)
        fprop()
        events[1].record(main)
        wgrad()
        events[2].record(main)
        dgrad()
        events[3].record(main)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    if _clib.device_status() != 0:
        raise SystemExit("kernel status word reported a wait time-out during warm-up")

    # ---- data-parallel parity: the summed dw of a 64-image global batch sharded over the ranks
    # equals the dw of the whole batch on one rank, and is identical on every rank
    dp_parity = None
    if world > 1:
        gb = 64
        g2 = torch.Generator(device="cpu").manual_seed(4321)
        gx = torch.randn(gb, C, H, W, generator=g2).half()
        gdy = torch.randn(gb, C, H, W, generator=g2).half()
        per = gb // world
        sx = gx[rank * per:(rank + 1) * per].to(dev).contiguous(memory_format=CL)
        sdy = gdy[rank * per:(rank + 1) * per].to(dev).contiguous(memory_format=CL)
        s_sh = _clib.Shape(per, C, H, W, R, S, PAD, PAD)
        sdx = torch.empty_like(sx)
        sdw = torch.empty_like(dw)
        backward(sx, sdy, sdx, sdw, ctypes.byref(s_sh))
        reduce_dw(sdw)
        torch.cuda.synchronize(dev)
        gathered = [torch.empty_like(sdw) for _ in range(world)]
        dist.all_gather(gathered, sdw)
        same = all(torch.equal(gathered[0], g) for g in gathered)
        err = 0.0
        if rank == 0:
            fx, fdy = gx.to(dev).contiguous(memory_format=CL), gdy.to(dev).contiguous(memory_format=CL)
            f_sh = _clib.Shape(gb, C, H, W, R, S, PAD, PAD)
            fdw = torch.empty_like(dw)
            nb = lib.spio_conv2d_gw8_wgrad_scratch_bytes(ctypes.byref(f_sh), None)
            fs = torch.empty(nb, dtype=torch.uint8, device=dev)
            _clib.check(lib.spio_conv2d_gw8_wgrad(fdw.data_ptr(), fx.data_ptr(), fdy.data_ptr(), ctypes.byref(f_sh),
                                                  None, fs.data_ptr(), nb, sp))
            torch.cuda.synchronize(dev)
            err = float((fdw - sdw).abs().max() / fdw.abs().max())
        flag = torch.tensor([1 if (same and err <= 1e-5) else 0], device=dev)
        dist.broadcast(flag, 0)
        if int(flag.item()) != 1:
            raise SystemExit(f"data-parallel parity failed: identical on all ranks = {same}, "
                             f"relative difference to the single-rank weight gradient = {err:.3g}")
        dp_parity = "ok"
        barrier()

    sampler = ClockSampler(local_rank, period_s=0.0005)
    if rank == 0:
        sampler.start()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record(main)
    for k in range(args.steps):
        step()
    t1.record(main)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t0.elapsed_time(t1)
    if _clib.device_status() != 0:
        raise SystemExit("kernel status word reported a wait time-out")

    # ---- second pass, outside the timed region: the same steps with an event between the
    # kernels, for the per-kernel durations (the event records themselves cost a few us per step)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(4)] for _ in range(args.steps)]
    for k in range(args.steps):
        step(evs[k])
    barrier()
    kern_ms = [statistics.fmean(e[i].elapsed_time(e[i + 1]) for e in evs) for i in range(3)]

    # a clean reference of the step's results for the end-to-end check below
    fprop()
    backward()
    reduce_dw()
    torch.cuda.synchronize(dev)

    # ---- end to end through the host-buffer C ABI: pinned host operands, H2D + D2H inside
    e2e_steps = 0 if args.no_e2e else min(args.steps, 3)
    act_bytes = n * C * H * W * 2
    e2e_s, e2e_ok, ceiling = float("nan"), None, None
    if e2e_steps:
        hx = torch.empty(n, H, W, C, dtype=torch.float16).pin_memory()
        hdy = torch.empty(n, H, W, C, dtype=torch.float16).pin_memory()
        hy = torch.empty(n, H, W, C, dtype=torch.float16).pin_memory()
        hdx = torch.empty(n, H, W, C, dtype=torch.float16).pin_memory()
        hw = torch.empty(C, R, S, 8, dtype=torch.float16).pin_memory()
        hdw = torch.empty(C, R, S, 8, dtype=torch.float32).pin_memory()
        hx.copy_(x.permute(0, 2, 3, 1))
        hdy.copy_(dy.permute(0, 2, 3, 1))
        hw.copy_(w.permute(0, 2, 3, 1))
        dwd = torch.empty(C, R, S, 8, dtype=torch.float32, device=dev)

        def e2e_step():
            # one library call: x and dy go up once in pieces, fprop / dgrad run as the pieces arrive,
            # y / dx come back while later pieces are still uploading; the weight gradient of the rank's
            # images is summed over the ranks on the device before it comes back
            dp = px.options() if px is not None else None
            _clib.check(lib.spio_conv2d_gw8_step_host_dp(
                hy.data_ptr(), hdx.data_ptr(), hdw.data_ptr(), None, hx.data_ptr(), hdy.data_ptr(), hw.data_ptr(),
                None, shp, ctypes.byref(dp) if dp is not None else None))
            if px is not None:
                px.advance()
            elif world > 1:   # NCCL route: sum on the device, result back to the host buffer
                dwd.copy_(hdw, non_blocking=True)
                dist.all_reduce(dwd)
                hdw.copy_(dwd)

        e2e_step()
        barrier()
        w0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_s = (time.perf_counter() - w0) / e2e_steps
        # the host-buffer results must equal the device-pointer results: every element of y, dx and dw
        e2e_ok = bool(torch.equal(hy, y.permute(0, 2, 3, 1).cpu()) and torch.equal(hdx, dx.permute(0, 2, 3, 1).cpu()))
        dw_host, dw_dev = hdw, dw.permute(0, 2, 3, 1).cpu()
        e2e_ok = e2e_ok and bool(torch.equal(dw_host, dw_dev) if (world == 1 or px is not None)
                                 else torch.allclose(dw_host, dw_dev, rtol=1e-5, atol=1e-3))
        if world > 1:   # and the returned dw is the same on every rank
            parts = [torch.empty_like(dwd) for _ in range(world)]
            dist.all_gather(parts, hdw.to(dev))
            e2e_ok = e2e_ok and all(torch.equal(parts[0], p) for p in parts)
        ceiling = copy_ceiling(dev, world, dist)

    # ---- sustained: a few hundred steps, long enough for the power management to settle (after the
    # short measurements, which it would otherwise disturb: the clock sags for a while afterwards)
    sus_steps = max(200, args.steps) if not args.no_sustained else 0
    sus_ms, sus_clocks = float("nan"), None
    if sus_steps:
        s2 = ClockSampler(local_rank)
        if rank == 0:
            s2.start()
        barrier()
        t0.record(main)
        for k in range(sus_steps):
            step()
        t1.record(main)
        barrier()
        sus_clocks = s2.stop() if rank == 0 else None
        sus_ms = t0.elapsed_time(t1) / sus_steps

    times = torch.tensor([total_ms, e2e_s * 1e3, sus_ms] + kern_ms, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, sus_ms, k_fprop, k_wgrad, k_dgrad = times.tolist()

    if rank == 0:
        ms_per_step = total_ms / args.steps
        b_one = algorithmic_bytes(n)
        step_bytes_all = 3 * b_one * world
        GB = global_batch
        peak, peak_kind = measured_peak()
        achieved = b_one / (k_fprop * 1e-3) / 1e9
        launches_per_step = 4 + (1 if px is not None else 0)
        wl = (f"cfg5 DP gw8 train step: C=K=64 56x56 3x3 pad1 gw8 fp16 NHWC, global batch "
              f"{GB} sharded over {world} GPU(s) ({n}/rank); fprop+wgrad+dgrad"
              + (f", dw summed over the ranks: {collective}" if world > 1 else ""))
        h2d = 2 * act_bytes + C * R * S * 8 * 2
        d2h = 2 * act_bytes + C * R * S * 8 * 4
        line = {
            "metric": "gw8 conv fprop+dgrad+wgrad effective bandwidth (algorithmic bytes / device time)",
            "value": step_bytes_all / (ms_per_step * 1e-3) / 1e9,
            "unit": "GB/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "f16 operands, f32 accumulate",
            "data": "synthetic",
            "config": {"workload": wl, "global_batch": GB, "per_rank_batch": n,
                       "l2": "every streamed operand > L2 (126 MB); no flush between steps",
                       "parallelism": f"dp{world}", "collective": collective,
                       "tune": tunes or "planner defaults"},
            "images_per_s": GB / (ms_per_step * 1e-3),
            "frac_of_8TBps_nominal": step_bytes_all / world / (ms_per_step * 1e-3) / 1e9 / 8000.0,
            "dp_parity": dp_parity,
            "sustained": None if not sus_steps else {
                "steps": sus_steps, "ms_per_step": sus_ms,
                "value": step_bytes_all / (sus_ms * 1e-3) / 1e9, "unit": "GB/s", "clocks": sus_clocks},
            "kernels_note": "per-kernel times come from a second pass of the same steps with CUDA events "
                            "between the kernels, run after the timed region (no exchange in that pass)",
            "kernels": {
                name: {"ms": ms, "GBps": b_one / (ms * 1e-3) / 1e9, "frac_of_measured_peak": b_one / (ms * 1e-3) / 1e9 / peak}
                for name, ms in (("fprop", k_fprop), ("wgrad+reduce", k_wgrad), ("dgrad", k_dgrad))
            },
            "roofline": {"bound": "hbm", "kernel": "conv2d_gw8_fwd_kernel (fprop launch)",
                         "achieved": achieved, "peak": peak, "peak_kind": peak_kind + " copy bandwidth",
                         "unit": "GB/s", "frac": achieved / peak,
                         "traffic": fwd_dram_traffic(b_one),
                         "traffic_source": "ncu capture at N=512 scaled to this batch (profiles/)",
                         "algorithmic_bytes_per_launch": b_one},
            "e2e": None if not e2e_steps else {
                "value": step_bytes_all / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                "ms_per_step": e2e_ms, "steps": e2e_steps,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "copy_GBps": world * (h2d + d2h) / (e2e_ms * 1e-3) / 1e9,
                "copy_ceiling_gbs": ceiling,
                "frac_of_copy_ceiling": world * (h2d + d2h) / (e2e_ms * 1e-3) / 1e9 / ceiling if ceiling else None,
                "copy_ceiling_note": "plain pinned cudaMemcpyAsync, 256 MB up and 256 MB down per rank at the "
                                     "same time, all ranks at once, aggregate of both directions",
                "matches_device_path": e2e_ok,
                "api": "spio_conv2d_gw8_step_host_dp (pinned host buffers; uploads, kernels and downloads of the "
                       "batch pieces overlap on three streams; dw summed over the ranks on the device)"},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if world == 1 and not args.no_sweep:
            time.sleep(0.5)
            incumbent_ok = False
            if not args.no_incumbent:
                try:
                    from oracle import ref_kernels

                    incumbent_ok = ref_kernels.available()
                except Exception:
                    incumbent_ok = False
            line["incumbent_note"] = (
                "the reference's own kernels (spio/src/conv2d_gw8.cu, conv2d_gw8_wgrad.cu) NVRTC-compiled for sm_100a "
                "from the reference checkout, best of the built configurations per kernel, launched as the reference "
                "launches them (no programmatic launch, zero fill before wgrad)" if incumbent_ok
                else "oracle/_ref has not been built: no incumbent figures")
            sweep = {}
            for bn in (128, 256, 512):
                pt = LayerPoint(lib, dev, bn, C, H, seed=1234 + 2)
                sweep[f"n{bn}"] = {"algorithmic_bytes": pt.bytes, "operand_sets": pt.sets,
                                   "c_abi_planner_defaults": pt.c_abi(), "operator_tuned_tables": pt.operator()}
                if incumbent_ok:
                    sweep[f"n{bn}"]["incumbent_reference_kernels"] = pt.incumbent()
                if not args.no_incumbent:
                    sweep[f"n{bn}"]["incumbent_torch_cudnn"] = pt.cudnn()
                del pt
                torch.cuda.empty_cache()
            line["sweep"] = sweep
            line["sweep_note"] = ("C=K=64 56x56 3x3 layer; us per launch in a chain of back-to-back launches rotating "
                                  "over operand sets > 600 MB (cold L2), programmatic dependent launch on; 'backward' is "
                                  "the combined call (wgrad, reduce, dgrad; rate over the bytes of two kernels); 'step' is "
                                  "fprop + combined backward, its rate counts the bytes of three kernels; operator = "
                                  "torch.ops.spio.conv2d_gw8 + autograd with the tuning-table configurations, timed on "
                                  "the device with the host queued ahead")
            ladder = {}
            for c_, hw_ in ((128, 56), (256, 28), (512, 14), (768, 7)):
                pt = LayerPoint(lib, dev, 256, c_, hw_, seed=1234 + 3)
                ladder[f"c{c_}_{hw_}x{hw_}"] = {"algorithmic_bytes": pt.bytes, "operand_sets": pt.sets,
                                                "c_abi_planner_defaults": pt.c_abi(), "operator_tuned_tables": pt.operator()}
                if incumbent_ok:
                    ladder[f"c{c_}_{hw_}x{hw_}"]["incumbent_reference_kernels"] = pt.incumbent()
                if not args.no_incumbent:
                    ladder[f"c{c_}_{hw_}x{hw_}"]["incumbent_torch_cudnn"] = pt.cudnn()
                del pt
                torch.cuda.empty_cache()
            line["ladder"] = ladder
            if incumbent_ok and global_batch == GLOBAL_BATCH:   # last: the heaviest leg
                time.sleep(0.5)
                pt = LayerPoint(lib, dev, global_batch, C, H, seed=1234 + 5)
                line["incumbent"] = pt.incumbent(count=8)
                ours_step = pt.c_abi(count=8)["step"]["us"]
                line["incumbent"]["ours_step_us_same_protocol"] = ours_step
                if "step" in line["incumbent"]:
                    line["incumbent"]["speedup_of_step"] = line["incumbent"]["step"]["us"] / ours_step
                del pt
                torch.cuda.empty_cache()
            line["host_us_per_call"] = sweep["n256"]["c_abi_planner_defaults"]["host_us_per_call"]
            if not args.no_convnext:
                try:
                    line["convnext_step_ms"] = convnext_step_ms(dev)
                    if not args.no_incumbent:
                        line["convnext_step_ms"]["stock_torch_ms"] = convnext_step_ms(dev, stock=True)["ms"]
                except Exception as exc:  # the headline must not depend on the example model
                    line["convnext_step_ms"] = {"error": str(exc)[:200]}
            if _clib.device_status() != 0:
                raise SystemExit("kernel status word reported a wait time-out in the sweeps")
        line["cpu_baseline"] = cpu_baseline(max_seconds=20.0) if world == 1 and not args.no_cpu else None
        print(json.dumps(line), flush=True)
    if px_all is not None or px is not None:
        barrier()
        (px_all or px).close()
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------ CPU arm

def cpu_step_time(n: int, reps: int):
    """Best-of-reps seconds of fprop + (dgrad, wgrad) on n images with torch's CPU conv2d,
    fp32 on fp16-rounded operands: the function the reference's tests use as their oracle."""
    from oracle import oracle as O

    sh = O.Shape(n, C, H, W, R, S, PAD, PAD)
    x, w, _, dy = O.make_inputs(sh, seed=1234 + 5, bias=False)
    x, dy = x.contiguous(memory_format=CL), dy.contiguous(memory_format=CL)
    best = float("inf")
    for _ in range(reps + 1):
        t = time.perf_counter()
        O.torch_fprop(x, w, None, sh)
        O.torch_grads(x, w, dy, sh)
        best = min(best, time.perf_counter() - t)
    return best


def use_all_host_cores() -> int:
    """torch.distributed.run sets OMP_NUM_THREADS=1 for its workers; the CPU arm is meant to use
    every host core, so the thread count is set explicitly and reported."""
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    return torch.get_num_threads()


def cpu_baseline(max_seconds: float = 20.0) -> dict:
    threads = use_all_host_cores()
    n = 16
    t = cpu_step_time(n, reps=1)
    while t * 4 < max_seconds / 3 and n < 256:
        n *= 2
        t = cpu_step_time(n, reps=1)
    t = min(t, cpu_step_time(n, reps=2))
    b = 3 * algorithmic_bytes(n)
    return {"value": b / t / 1e9, "unit": "GB/s", "cores": threads,
            "host_cpus": os.cpu_count(), "kind": "port", "images_per_s": n / t,
            "sample": (f"{n} images of the same layer, fprop + dgrad + wgrad, best of 3; "
                       "torch.nn.functional.conv2d fp32 + autograd on the host cores (the reference "
                       "has no CPU kernels; this is the oracle its tests compare against)")}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    threads = use_all_host_cores()
    n = 32
    warm = max(args.warmup, 1)
    for _ in range(min(warm, 5)):
        cpu_step_time(n, reps=0)
    times = [cpu_step_time(n, reps=0) for _ in range(max(1, args.steps))]
    t = statistics.fmean(times)
    b = 3 * algorithmic_bytes(n)
    val = b / t / 1e9
    sample = (f"{n} images per step of the C=64 56x56 3x3 gw8 layer (bounded sample of the "
              f"{GLOBAL_BATCH}-image workload), fprop + dgrad + wgrad with torch CPU conv2d fp32")
    line = {
        "impl": "reference",
        "metric": "gw8 conv fprop+dgrad+wgrad effective bandwidth (algorithmic bytes / device time)",
        "value": val, "unit": "GB/s", "n_gpus": world, "steps": len(times), "warmup": warm,
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 on f16-rounded operands", "data": "synthetic",
        "config": {"workload": sample, "parallelism": f"host cores ({threads} threads)"},
        "images_per_s": n / t,
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads,
                         "host_cpus": os.cpu_count(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--no-sweep", action="store_true", help="skip the batch sweep, the ladder and the ConvNeXt step")
    ap.add_argument("--no-convnext", action="store_true", help="skip the ConvNeXt train step")
    ap.add_argument("--no-sustained", action="store_true", help="skip the 200-step run")
    ap.add_argument("--no-incumbent", action="store_true", help="skip the reference's own kernels")
    ap.add_argument("--collective", choices=["auto", "peer", "nccl"], default="auto",
                    help="how dw is summed over the ranks (N > 1); auto = the peer-store exchange inside the launch "
                         "chain, NCCL if it cannot be set up")
    ap.add_argument("--force-exchange", action="store_true",
                    help="1 GPU: run the peer-store exchange with the rank itself")
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH,
                    help="images over all ranks (default: the 2048 of the data-parallel sweep)")
    ap.add_argument("--tune", default="",
                    help='JSON overrides of the launch plans, e.g. \'{"fprop": {"pps": 1}, "wgrad": {"ns": 4}}\'')
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
