"""The data-parallel sum of the weight gradient by peer stores (spio_dp_push / spio_dp_sum).

One GPU is enough to check the kernels' bookkeeping: the "ranks" are buffers of one device and
all pushes of an exchange are queued before its sums, so no kernel ever waits for one that has
not been launched (on one GPU that could never be satisfied).  The two-process test runs the
real thing -- one process per GPU, IPC-mapped buffers, the exchange inside the combined
backward call -- and is skipped on a single-GPU machine.
"""

import ctypes
import os
import socket

import pytest
import torch

from oracle import oracle as O
from spio_b200 import _clib
from tests import capi

pytestmark = pytest.mark.gpu


def alloc_buffers(world, capacity):
    lib = _clib.load()
    nbytes = lib.spio_dp_buffer_bytes(world, capacity)
    assert nbytes >= 256 + 2 * world * capacity * 8   # a word is {float, tag}
    bufs = []
    for _ in range(world):
        p = ctypes.c_void_p()
        _clib.check(lib.spio_dp_buffer_alloc(nbytes, ctypes.byref(p), None))
        bufs.append(p)
    table = (ctypes.c_void_p * world)(*[b.value for b in bufs])
    return bufs, table


def exchange(table, rank, world, seq, capacity):
    return _clib.DpExchange(ctypes.cast(table, ctypes.POINTER(ctypes.c_void_p)), rank, world, seq, capacity)


def test_allreduce_of_one_rank_is_the_identity():
    lib = _clib.load()
    bufs, table = alloc_buffers(1, 4672)
    a = torch.randn(4608, device="cuda:0")
    b = torch.randn(64, device="cuda:0")
    keep = (a.clone(), b.clone())
    try:
        for seq in range(3):
            dp = exchange(table, 0, 1, seq, 4672)
            _clib.check(lib.spio_dp_allreduce(ctypes.byref(dp), a.data_ptr(), 4608, b.data_ptr(), 64,
                                              torch.cuda.current_stream().cuda_stream))
        assert torch.equal(a, keep[0]) and torch.equal(b, keep[1])
        assert capi.status() == 0
    finally:
        torch.cuda.synchronize()
        lib.spio_dp_buffer_free(bufs[0])


@pytest.mark.parametrize("world", [1, 2, 5, 8])
def test_rank_order_sum_over_emulated_ranks(world):
    from spio_b200.distributed import rank_order_sum

    lib = _clib.load()
    n_a, n_b, capacity = 4608, 64, 4672
    bufs, table = alloc_buffers(world, capacity)
    stream = torch.cuda.current_stream().cuda_stream
    gen = torch.Generator(device="cuda:0").manual_seed(7)
    try:
        for seq in range(5):   # both parities, flags counting up
            a = [torch.randn(n_a, device="cuda:0", generator=gen) for _ in range(world)]
            b = [torch.randn(n_b, device="cuda:0", generator=gen) for _ in range(world)]
            want_a, want_b = rank_order_sum(a), rank_order_sum(b)
            dps = [exchange(table, r, world, seq, capacity) for r in range(world)]
            for r in range(world):
                _clib.check(lib.spio_dp_push(ctypes.byref(dps[r]), a[r].data_ptr(), n_a, b[r].data_ptr(), n_b, stream))
            for r in range(world):
                _clib.check(lib.spio_dp_sum(ctypes.byref(dps[r]), a[r].data_ptr(), n_a, b[r].data_ptr(), n_b, stream))
            for r in range(world):   # bit-identical on every rank
                assert torch.equal(a[r], want_a) and torch.equal(b[r], want_b), f"seq {seq} rank {r}"
        assert capi.status() == 0
    finally:
        torch.cuda.synchronize()
        for p in bufs:
            lib.spio_dp_buffer_free(p)


def test_a_missing_peer_is_reported_not_waited_for_for_ever():
    """Rank 1 never pushes: rank 0's sum gives up after the wait limit (2 s), records
    SPIO_STATUS_PEER_TIMEOUT and leaves the vector alone; the device stays usable."""
    lib = _clib.load()
    bufs, table = alloc_buffers(2, 64)
    stream = torch.cuda.current_stream().cuda_stream
    a = torch.arange(64, dtype=torch.float32, device="cuda:0")
    keep = a.clone()
    try:
        dp = exchange(table, 0, 2, 0, 64)
        _clib.check(lib.spio_dp_push(ctypes.byref(dp), a.data_ptr(), 64, None, 0, stream))
        _clib.check(lib.spio_dp_sum(ctypes.byref(dp), a.data_ptr(), 64, None, 0, stream))
        assert capi.status() == 2
        assert capi.status() == 0
        assert torch.equal(a, keep)
    finally:
        torch.cuda.synchronize()
        for p in bufs:
            lib.spio_dp_buffer_free(p)
    sh = O.Shape(2, 64, 16, 16, 3, 3, 1, 1)
    x, w, b, _ = O.make_inputs(sh, seed=3, bias=True)
    xd, wd, bd = (capi.to_dev(t) for t in (x, w, b))
    O.assert_close(capi.fprop(xd, wd, bd, sh), O.c_fprop(x, w, b, sh), sh, "fprop", "after a peer time-out")


def test_bad_arguments_are_rejected():
    lib = _clib.load()
    assert lib.spio_dp_buffer_bytes(17, 64) == 0
    bufs, table = alloc_buffers(1, 64)
    a = torch.zeros(128, device="cuda:0")
    try:
        for dp, n in ((exchange(table, 0, 1, 0, 64), 128), (exchange(table, 1, 1, 0, 64), 64),
                      (exchange(table, 0, 1, 0, 64), 6)):
            assert lib.spio_dp_push(ctypes.byref(dp), a.data_ptr(), n, None, 0, None) != 0
            assert "data-parallel exchange" in _clib.last_error()
    finally:
        for p in bufs:
            lib.spio_dp_buffer_free(p)


def test_backward_with_the_exchange_on_one_rank():
    """world = 1: the chain wgrad -> reduce -> push -> dgrad -> sum gives the plain backward's bits."""
    lib = _clib.load()
    sh = O.Shape(16, 72, 28, 28, 3, 3, 1, 1)
    x, w, _, dy = O.make_inputs(sh, seed=31, bias=False)
    xd, wd, dyd = (capi.to_dev(t) for t in (x, w, dy))
    ref_dx, ref_dw, ref_db = capi.backward(xd, dyd, wd, sh, with_bias=True)
    capacity = sh.c * 72 + sh.c
    bufs, table = alloc_buffers(1, capacity)
    s = capi.cshape(sh)
    nbytes = lib.spio_conv2d_gw8_wgrad_scratch_bytes(ctypes.byref(s), None)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda:0")
    try:
        for seq in range(4):
            dx = torch.full_like(ref_dx, capi.DEAD_VALUE)
            dw = torch.full_like(ref_dw, capi.DEAD_VALUE)
            db = torch.full_like(ref_db, capi.DEAD_VALUE)
            dp = exchange(table, 0, 1, seq, capacity)
            opts = _clib.BackwardOpts(0, None, None, None, ctypes.pointer(dp))
            _clib.check(lib.spio_conv2d_gw8_backward_ex(
                dx.data_ptr(), dw.data_ptr(), db.data_ptr(), xd.data_ptr(), dyd.data_ptr(), wd.data_ptr(),
                ctypes.byref(s), None, None, scratch.data_ptr(), nbytes, torch.cuda.current_stream().cuda_stream,
                None, ctypes.byref(opts)))
            assert torch.equal(dx, ref_dx) and torch.equal(dw, ref_dw) and torch.equal(db, ref_db), f"seq {seq}"
        assert capi.status() == 0
    finally:
        torch.cuda.synchronize()
        for p in bufs:
            lib.spio_dp_buffer_free(p)


# ------------------------------------------------------------------ two processes, two GPUs

def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _dp_worker(rank: int, world: int, port: int, out_dir: str):
    import torch.distributed as dist

    from spio_b200.distributed import PeerExchange, shard_batch

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        dev = f"cuda:{rank}"
        lib = _clib.load()
        sh = O.Shape(64, 64, 28, 28, 3, 3, 1, 1)
        x, w, _, dy = O.make_inputs(sh, seed=1234 + 5, bias=False)   # the same global batch on every rank
        xs, dys = shard_batch(x, world, rank), shard_batch(dy, world, rank)
        sub = O.Shape(xs.shape[0], sh.c, sh.h, sh.w, sh.r, sh.s, sh.pad_h, sh.pad_w)
        xd, dyd, wd = capi.to_dev(xs, dev), capi.to_dev(dys, dev), capi.to_dev(w, dev)
        capacity = sh.c * 72 + sh.c
        px = PeerExchange(capacity, device=torch.device(dev))
        s = capi.cshape(sub)
        nbytes = lib.spio_conv2d_gw8_wgrad_scratch_bytes(ctypes.byref(s), None)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        results = []
        for step in range(6):
            dx = torch.full((sub.n, sub.c, sub.h, sub.w), capi.DEAD_VALUE, dtype=torch.float16, device=dev)
            dx = dx.contiguous(memory_format=capi.CL)
            dw = torch.full((sh.c, 8, 3, 3), capi.DEAD_VALUE, dtype=torch.float32, device=dev).contiguous(memory_format=capi.CL)
            db = torch.full((sh.c,), capi.DEAD_VALUE, dtype=torch.float32, device=dev)
            dp = px.options()
            opts = _clib.BackwardOpts(0, None, None, None, ctypes.pointer(dp))
            _clib.check(lib.spio_conv2d_gw8_backward_ex(
                dx.data_ptr(), dw.data_ptr(), db.data_ptr(), xd.data_ptr(), dyd.data_ptr(), wd.data_ptr(),
                ctypes.byref(s), None, None, scratch.data_ptr(), nbytes, torch.cuda.current_stream().cuda_stream,
                None, ctypes.byref(opts)))
            px.advance()
            results.append((dw, db, dx))
        torch.cuda.synchronize()
        status = _clib.device_status()
        torch.save({"dw": [r[0].cpu() for r in results], "db": [r[1].cpu() for r in results],
                    "dx": results[-1][2].cpu(), "status": status}, os.path.join(out_dir, f"rank{rank}.pt"))
        dist.barrier()
        px.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_data_parallel_backward(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_dp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = [torch.load(tmp_path / f"rank{r}.pt") for r in range(world)]
    sh = O.Shape(64, 64, 28, 28, 3, 3, 1, 1)
    x, w, _, dy = O.make_inputs(sh, seed=1234 + 5, bias=False)
    want_dw = O.c_wgrad(x, dy, sh)
    for r in range(world):
        assert got[r]["status"] == 0
    for step in range(6):
        assert torch.equal(got[0]["dw"][step], got[1]["dw"][step])      # bit-identical on both ranks
        assert torch.equal(got[0]["db"][step], got[1]["db"][step])
        assert torch.equal(got[0]["dw"][step], got[0]["dw"][0])         # and from step to step
        O.assert_close(got[0]["dw"][step], want_dw, sh, "wgrad", f"2-GPU sum, step {step}")
        torch.testing.assert_close(got[0]["db"][step], dy.float().sum(dim=(0, 2, 3)), rtol=1e-3, atol=5e-2)
    O.assert_close(torch.cat([got[0]["dx"], got[1]["dx"]]), O.c_dgrad(dy, w, sh), sh, "dgrad", "2-GPU shards")
