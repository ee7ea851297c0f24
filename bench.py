"""Benchmark of the gw8 convolution training step (fprop + wgrad + dgrad) on B200.

    python bench.py --gpus N --steps K --warmup W            # this package's CUDA kernels
    python bench.py --impl reference --gpus N ...            # CPU baseline arm

Workload (default): the data-parallel sweep layer -- C=K=64, 56x56, 3x3, stride 1, pad 1,
group width 8, fp16 NHWC -- with a GLOBAL batch of 2048 images sharded over the N ranks
(strong scaling).  One step = forward, weight gradient, input gradient on the rank's
shard; with N > 1 the fp32 weight gradient is summed with one NCCL all-reduce that
overlaps the input-gradient kernel.  Synthetic seeded N(0,1) activations / gradients and
N(0, 1/sqrt(72)) weights.  Every operand streamed by a kernel is larger than the 126 MB L2
at every N (>= 205 MB per kernel launch at N=8), so no L2 flush is needed between steps.

Prints ONE JSON line (rank 0).  ``value`` is whole-job effective bandwidth: algorithmic
bytes of the three kernels over all ranks (spio_b200.kernels.Conv2dStats, 2 bytes per
element, each operand once) divided by the device time of a step, max over ranks.
"""

from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GLOBAL_BATCH = 2048
C, H, W, R, S, PAD = 64, 56, 56, 3, 3, 1
L2_BYTES = 126 * 1024 * 1024
# DRAM traffic of one forward-kernel launch, from the ncu capture at N=512 summarised in
# profiles/conv2d_gw8_fwd_kernel__c64_56x56_3x3_n512.md: reads are 1.010 x the input bytes
# (halo rows at span ends); writes are the output bytes minus ~50 MB that are still dirty in
# the 126 MB L2 when the kernel ends.  Reads and writes grow with the batch, the L2 residue
# does not, so a launch at another batch is estimated as below.
FWD_DRAM_READ_RATIO = 1.015
FWD_L2_RESIDUE_BYTES = 47.7e6


def fwd_dram_traffic(algorithmic: int) -> float:
    half = algorithmic / 2.0
    return FWD_DRAM_READ_RATIO * half + max(half - FWD_L2_RESIDUE_BYTES, 0.0)


def algorithmic_bytes(n: int) -> int:
    """Bytes of ONE of the three kernels for a batch of n (identical for all three)."""
    from spio_b200.kernels import Conv2dGw8Params, Conv2dStats

    return Conv2dStats(Conv2dGw8Params(n=n, c=C, h=H, w=W, padding=PAD, r=R, s=S),
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

    def __init__(self, index: int, period_s: float = 0.003):
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


# ------------------------------------------------------------------------------ our arm

def run_ours(args) -> None:
    import torch.distributed as dist

    from spio_b200 import _clib
    from spio_b200.kernels import Conv2dGw8Params

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
    cl = torch.channels_last
    x = torch.randn(n, C, H, W, device=dev, generator=gen).half().contiguous(memory_format=cl)
    dy = torch.randn(n, C, H, W, device=dev, generator=gen).half().contiguous(memory_format=cl)
    wgen = torch.Generator(device=dev).manual_seed(1234 + 5)
    w = (torch.randn(C, 8, R, S, device=dev, generator=wgen) / 72 ** 0.5).half().contiguous(memory_format=cl)
    y = torch.empty_like(x)
    dx = torch.empty_like(x)
    dw = torch.empty(C, 8, R, S, device=dev, dtype=torch.float32).contiguous(memory_format=cl)

    main = torch.cuda.current_stream(dev)
    comm = torch.cuda.Stream(dev) if world > 1 else None
    sp = main.cuda_stream

    # Rank-local dgrad leaves one SM to the all-reduce kernel, which otherwise could not become
    # resident beside the persistent CTAs (one per SM) until they exit.
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    tunes = json.loads(args.tune) if args.tune else {}
    dgrad_cfg = dict(tunes.get("dgrad", {}))
    if world > 1:
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

    def fprop():
        _clib.check(lib.spio_conv2d_gw8_fprop(y.data_ptr(), x.data_ptr(), w.data_ptr(), None, shp, fprop_tp, sp))

    def wgrad():
        _clib.check(lib.spio_conv2d_gw8_wgrad(dw.data_ptr(), x.data_ptr(), dy.data_ptr(), shp, wgrad_tp,
                                              scratch.data_ptr(), scratch_bytes, sp))

    def dgrad():
        _clib.check(lib.spio_conv2d_gw8_dgrad(dx.data_ptr(), dy.data_ptr(), w.data_ptr(), shp, dgrad_tp, sp))

    def backward():
        # wgrad -> reduce -> (dw_ready) -> dgrad, chained with programmatic dependent launch
        _clib.check(lib.spio_conv2d_gw8_backward(
            dx.data_ptr(), dw.data_ptr(), None, x.data_ptr(), dy.data_ptr(), w.data_ptr(), shp, dgrad_tp, wgrad_tp,
            scratch.data_ptr(), scratch_bytes, sp, dw_ready.cuda_event if comm is not None else None))

    def step(events=None):
        """One training step of the layer.  With `events` the three kernels are launched
        separately so that each can be timed; otherwise backward is one library call."""
        if events is None:
            fprop()
            backward()
            if comm is not None:
                comm.wait_event(dw_ready)
                with torch.cuda.stream(comm):
                    dist.all_reduce(dw)
                main.wait_stream(comm)
            return
        events[0].record(main)
        fprop()
        events[1].record(main)
        wgrad()
        events[2].record(main)
        if comm is not None:
            comm.wait_stream(main)
            with torch.cuda.stream(comm):
                dist.all_reduce(dw)
        dgrad()
        events[3].record(main)
        if comm is not None:
            main.wait_stream(comm)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    if _clib.device_status() != 0:
        raise SystemExit("kernel status word reported a wait time-out during warm-up")

    sampler = ClockSampler(local_rank)
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

    # ---- end to end through the host-buffer C ABI: pinned host operands, H2D + D2H inside
    e2e_steps = 0 if args.no_e2e else min(args.steps, 3)
    act_bytes = n * C * H * W * 2
    e2e_s, e2e_ok = float("nan"), None
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

        def e2e_step():
            # one library call: x and dy go up once in pieces, fprop / dgrad / wgrad run as the
            # pieces arrive, y / dx / dw come back while later pieces are still uploading
            _clib.check(lib.spio_conv2d_gw8_step_host(hy.data_ptr(), hdx.data_ptr(), hdw.data_ptr(), None,
                                                      hx.data_ptr(), hdy.data_ptr(), hw.data_ptr(), None, shp))

        e2e_step()
        barrier()
        w0 = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_step()
        barrier()
        e2e_s = (time.perf_counter() - w0) / e2e_steps
        # the host-buffer result must equal the device-pointer result bit for bit
        e2e_ok = bool(torch.equal(hy[:2], y[:2].permute(0, 2, 3, 1).cpu()))

    times = torch.tensor([total_ms, e2e_s * 1e3] + kern_ms, device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    total_ms, e2e_ms, k_fprop, k_wgrad, k_dgrad = times.tolist()

    if rank == 0:
        ms_per_step = total_ms / args.steps
        b_one = algorithmic_bytes(n)
        step_bytes_all = 3 * b_one * world
        GB = global_batch
        peak, peak_kind = measured_peak()
        achieved = b_one / (k_fprop * 1e-3) / 1e9
        wl = (f"cfg5 DP gw8 train step: C=K=64 56x56 3x3 pad1 gw8 fp16 NHWC, global batch "
              f"{GB} sharded over {world} GPU(s) ({n}/rank); fprop+wgrad+dgrad"
              + (", 1 NCCL all-reduce of dw overlapped with dgrad (dgrad on all SMs but one)" if world > 1 else ""))
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
                       "parallelism": f"dp{world}", "tune": tunes or "planner defaults"},
            "images_per_s": GB / (ms_per_step * 1e-3),
            "frac_of_8TBps_nominal": step_bytes_all / world / (ms_per_step * 1e-3) / 1e9 / 8000.0,
            "kernels_note": "per-kernel times come from a second pass of the same steps with CUDA events "
                            "between the kernels, run after the timed region",
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
            "e2e": None if not e2e_steps else {"value": step_bytes_all / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
                    "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "h2d_bytes_per_step": 2 * act_bytes + C * R * S * 8 * 2,
                    "d2h_bytes_per_step": 2 * act_bytes + C * R * S * 8 * 4,
                    "matches_device_path": e2e_ok,
                    "api": "spio_conv2d_gw8_step_host (pinned host buffers; uploads, kernels and downloads "
                           "of 32 pieces of the batch overlap on three streams)"},
            "gpu_launches": 4 * args.steps,
            "clocks": clocks,
        }
        line["cpu_baseline"] = cpu_baseline(max_seconds=20.0) if world == 1 and not args.no_cpu else None
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------------------------ CPU arm

def cpu_step_time(n: int, reps: int):
    """Best-of-reps seconds of fprop + (dgrad, wgrad) on n images with torch's CPU conv2d,
    fp32 on fp16-rounded operands: the function the reference's tests use as their oracle."""
    from oracle import oracle as O

    sh = O.Shape(n, C, H, W, R, S, PAD, PAD)
    x, w, _, dy = O.make_inputs(sh, seed=1234 + 5, bias=False)
    cl = torch.channels_last
    x, dy = x.contiguous(memory_format=cl), dy.contiguous(memory_format=cl)
    best = float("inf")
    for _ in range(reps + 1):
        t = time.perf_counter()
        O.torch_fprop(x, w, None, sh)
        O.torch_grads(x, w, dy, sh)
        best = min(best, time.perf_counter() - t)
    return best


def cpu_baseline(max_seconds: float = 20.0) -> dict:
    n = 16
    t = cpu_step_time(n, reps=1)
    while t * 4 < max_seconds / 3 and n < 256:
        n *= 2
        t = cpu_step_time(n, reps=1)
    t = min(t, cpu_step_time(n, reps=2))
    b = 3 * algorithmic_bytes(n)
    return {"value": b / t / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(),
            "host_cpus": os.cpu_count(), "kind": "port", "images_per_s": n / t,
            "sample": (f"{n} images of the same layer, fprop + dgrad + wgrad, best of 3; "
                       "torch.nn.functional.conv2d fp32 + autograd on the host cores (the reference "
                       "has no CPU kernels; this is the oracle its tests compare against)")}


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    n = 32
    for _ in range(max(args.warmup, 1)):
        cpu_step_time(n, reps=0)
    times = [cpu_step_time(n, reps=0) for _ in range(max(1, min(args.steps, 10)))]
    t = statistics.fmean(times)
    b = 3 * algorithmic_bytes(n)
    val = b / t / 1e9
    sample = (f"{n} images per step of the C=64 56x56 3x3 gw8 layer (bounded sample of the "
              f"{GLOBAL_BATCH}-image workload), fprop + dgrad + wgrad with torch CPU conv2d fp32")
    line = {
        "impl": "reference",
        "metric": "gw8 conv fprop+dgrad+wgrad effective bandwidth (algorithmic bytes / device time)",
        "value": val, "unit": "GB/s", "n_gpus": world, "steps": len(times), "warmup": max(args.warmup, 1),
        "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32 on f16-rounded operands", "data": "synthetic",
        "config": {"workload": sample, "parallelism": "host cores"},
        "images_per_s": n / t,
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": torch.get_num_threads(),
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
