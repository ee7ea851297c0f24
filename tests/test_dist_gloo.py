"""The data-parallel path on CPU ranks (gloo, world size 2): sharding the seeded global batch
and summing the per-rank weight-gradient partials reproduces the single-process result."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from spio_b200.distributed import GradWeightReducer, rank_order_sum, shard_batch, shard_range


def test_shard_ranges_cover_the_batch():
    for n in (1, 7, 2048):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(8, 2, 2)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        O.set_num_threads(2)
        sh = O.Shape(6, 16, 9, 8, 3, 3, 1, 1)
        x, w, _, dy = O.make_inputs(sh, seed=1234 + 5, bias=False)   # same global batch on every rank
        xs, dys = shard_batch(x, world, rank), shard_batch(dy, world, rank)
        sub = O.Shape(xs.shape[0], sh.c, sh.h, sh.w, sh.r, sh.s, sh.pad_h, sh.pad_w)
        y_local = O.c_fprop(xs, w, None, sub)
        dx_local = O.c_dgrad(dys, w, sub)
        dw = O.c_wgrad(xs, dys, sub).contiguous()
        red = GradWeightReducer()
        red.start(dw)
        red.finish()
        # forward / input gradient need no exchange: gather only to compare
        ys = [torch.empty_like(y_local) for _ in range(world)]
        dxs = [torch.empty_like(dx_local) for _ in range(world)]
        dist.all_gather(ys, y_local.contiguous())
        dist.all_gather(dxs, dx_local.contiguous())
        # the order of the peer-store exchange: every rank holds every rank's partial and adds
        # them in rank order, so all ranks get the same bits whatever the arrival order was
        mine = O.c_wgrad(xs, dys, sub).contiguous()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        ordered = rank_order_sum(parts[::-1][::-1])
        torch.save({"ordered": ordered}, os.path.join(out_dir, f"ordered{rank}.pt"))
        if rank == 0:
            torch.save({"dw": dw, "y": torch.cat(ys), "dx": torch.cat(dxs)}, os.path.join(out_dir, "out.pt"))
    finally:
        dist.destroy_process_group()


def test_two_rank_data_parallel_matches_single_process(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = torch.load(tmp_path / "out.pt")
    sh = O.Shape(6, 16, 9, 8, 3, 3, 1, 1)
    x, w, _, dy = O.make_inputs(sh, seed=1234 + 5, bias=False)
    assert torch.equal(got["y"], O.c_fprop(x, w, None, sh))
    assert torch.equal(got["dx"], O.c_dgrad(dy, w, sh))
    O.assert_close(got["dw"], O.c_wgrad(x, dy, sh), sh, "wgrad", "2-rank sum")
    ordered = [torch.load(tmp_path / f"ordered{r}.pt")["ordered"] for r in range(world)]
    assert torch.equal(ordered[0], ordered[1])
    O.assert_close(ordered[0], O.c_wgrad(x, dy, sh), sh, "wgrad", "rank-order sum")
