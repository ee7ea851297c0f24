"""Full-size checks at the headline configurations, where the CPU oracle is too slow to
compute whole tensors: exact properties of the kernels plus oracle checks on slices.

* images are independent: the result for a slice of the batch equals the slice of the result
  (bit-exact), so the oracle needs only a few images;
* scaling an operand by a power of two scales the result exactly (fp16/fp32 arithmetic);
* the weight gradient is additive over the batch (fp32 reassociation tolerance) and equals a
  float64 reduction computed with torch on the device;
* the host-buffer entry points give bit-identical results to the device-pointer ones.
"""

import pytest
import torch

from oracle import oracle as O
from tests import capi

pytestmark = pytest.mark.gpu

FULL = [O.Shape(512, 64, 56, 56, 3, 3, 1, 1), O.Shape(256, 128, 56, 56, 3, 3, 1, 1),
        O.Shape(256, 256, 28, 28, 3, 3, 1, 1), O.Shape(256, 512, 14, 14, 3, 3, 1, 1),
        O.Shape(256, 768, 7, 7, 3, 3, 1, 1)]


def device_inputs(sh, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    cl = torch.channels_last
    x = torch.randn(sh.n, sh.c, sh.h, sh.w, device="cuda", generator=g).half().contiguous(memory_format=cl)
    dy = torch.randn(sh.n, sh.c, sh.p, sh.q, device="cuda", generator=g).half().contiguous(memory_format=cl)
    w = (torch.randn(sh.c, 8, sh.r, sh.s, device="cuda", generator=g) / (8 * sh.r * sh.s) ** 0.5)
    return x, w.half().contiguous(memory_format=cl), dy


@pytest.mark.parametrize("sh", FULL, ids=lambda s: f"n{s.n}c{s.c}hw{s.h}")
def test_full_size_slices_against_oracle(sh):
    x, w, dy = device_inputs(sh, seed=99)
    y = capi.fprop(x, w, None, sh)
    dx = capi.dgrad(dy, w, sh)
    assert capi.status() == 0
    assert not bool((y == capi.DEAD_VALUE).all(dim=1).any()), "unwritten output pixels"
    picks = [0, sh.n // 2 + 1, sh.n - 1]
    sub = O.Shape(len(picks), sh.c, sh.h, sh.w, sh.r, sh.s, sh.pad_h, sh.pad_w)
    xs, dys = x[picks].cpu(), dy[picks].cpu()
    O.assert_close(y[picks], O.c_fprop(xs, w.cpu(), None, sub), sub, "fprop", str(sh))
    O.assert_close(dx[picks], O.c_dgrad(dys, w.cpu(), sub), sub, "dgrad", str(sh))
    # batch independence, bit-exact: rerun on the slice alone
    ys = capi.fprop(x[picks].contiguous(memory_format=torch.channels_last), w, None, sub)
    assert torch.equal(ys, y[picks])


@pytest.mark.parametrize("sh", FULL[:2] + FULL[-1:], ids=lambda s: f"n{s.n}c{s.c}hw{s.h}")
def test_power_of_two_scaling_is_exact(sh):
    x, w, dy = device_inputs(sh, seed=100)
    y1 = capi.fprop(x, w, None, sh)
    y2 = capi.fprop(x * 2, w, None, sh)
    big = y1.abs() > 1e-3  # results in the fp16 subnormal range round differently
    assert torch.equal(y2[big], (y1 * 2)[big])
    d1 = capi.dgrad(dy, w, sh)
    d2 = capi.dgrad(dy * 2, w, sh)
    big = d1.abs() > 1e-3
    assert torch.equal(d2[big], (d1 * 2)[big])
    g1 = capi.wgrad(x, dy, sh)
    g2 = capi.wgrad(x * 2, dy * 2, sh)
    assert torch.equal(g2, g1 * 4)
    assert capi.status() == 0


@pytest.mark.parametrize("sh", FULL, ids=lambda s: f"n{s.n}c{s.c}hw{s.h}")
def test_full_size_wgrad(sh):
    x, w, dy = device_inputs(sh, seed=101)
    dw = capi.wgrad(x, dy, sh)
    assert capi.status() == 0
    # float64 reference on the device: dw[k,c,r,s] = sum x_shift[.., 8g+c] * dy[.., k]
    xp = torch.nn.functional.pad(x.double(), (sh.pad_w, sh.pad_w, sh.pad_h, sh.pad_h))
    ref = torch.empty(sh.c, 8, sh.r, sh.s, dtype=torch.float64, device="cuda")
    dyg = dy.double().view(sh.n, sh.c // 8, 8, sh.p, sh.q)
    for r in range(sh.r):
        for s in range(sh.s):
            xs = xp[:, :, r:r + sh.p, s:s + sh.q].reshape(sh.n, sh.c // 8, 8, sh.p, sh.q)
            ref[:, :, r, s] = torch.einsum("ngcpq,ngkpq->gkc", xs, dyg).reshape(sh.c, 8)
    O.assert_close(dw, ref.float(), sh, "wgrad", str(sh))
    # additivity over a split of the batch
    h = sh.n // 2
    half = O.Shape(h, sh.c, sh.h, sh.w, sh.r, sh.s, sh.pad_h, sh.pad_w)
    parts = capi.wgrad(x[:h], dy[:h], half) + capi.wgrad(x[h:], dy[h:], half)
    O.assert_close(parts, ref.float(), sh, "wgrad", f"{sh} split")


def test_host_buffer_entry_points_match_device_entry_points():
    import ctypes
    from spio_b200 import _clib

    sh = O.Shape(32, 64, 56, 56, 3, 3, 1, 1)
    x, w, b, dy = O.make_inputs(sh, seed=3, bias=True)
    lib = _clib.load()
    s = capi.cshape(sh)
    hx, hw, hdy = (O.nhwc(t).pin_memory() for t in (x, w, dy))
    hb = b.contiguous().pin_memory()
    hy = torch.empty(sh.n, sh.p, sh.q, sh.c, dtype=torch.float16).pin_memory()
    hdx = torch.empty(sh.n, sh.h, sh.w, sh.c, dtype=torch.float16).pin_memory()
    hdw = torch.empty(sh.c, sh.r, sh.s, 8, dtype=torch.float32).pin_memory()
    _clib.check(lib.spio_conv2d_gw8_fprop_host(hy.data_ptr(), hx.data_ptr(), hw.data_ptr(), hb.data_ptr(),
                                               ctypes.byref(s), None))
    _clib.check(lib.spio_conv2d_gw8_dgrad_host(hdx.data_ptr(), hdy.data_ptr(), hw.data_ptr(),
                                               ctypes.byref(s), None))
    _clib.check(lib.spio_conv2d_gw8_wgrad_host(hdw.data_ptr(), hx.data_ptr(), hdy.data_ptr(),
                                               ctypes.byref(s), None))
    xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
    assert torch.equal(O.from_nhwc(hy), capi.fprop(xd, wd, bd, sh).cpu())
    assert torch.equal(O.from_nhwc(hdx), capi.dgrad(dyd, wd, sh).cpu())
    assert torch.equal(O.from_nhwc(hdw), capi.wgrad(xd, dyd, sh).cpu())
    assert capi.status() == 0


def test_dynamic_tail_gives_identical_results():
    """The forward kernel's load warps claim the tail of the work from a global pool, in pieces
    of at most SPIO_DYN pairs that shrink as the pool drains (default 7, 0 = off; used from
    SPIO_DYN_MIN_PAIRS pairs per CTA).  The settings are read once per process, so the comparison
    runs in child processes: fprop and dgrad must be bit-identical with and without it, with the
    pool in use and over repeated launches (the counters are reused)."""
    import os
    import subprocess
    import sys
    import textwrap

    code = textwrap.dedent("""
        import sys, torch
        from oracle import oracle as O
        from tests import capi
        sh = O.Shape(96, 72, 56, 56, 3, 3, 1, 1)
        x, w, b, dy = O.make_inputs(sh, seed=31, bias=True)
        xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
        outs = []
        for _ in range(5):
            outs.append((capi.fprop(xd, wd, bd, sh), capi.dgrad(dyd, wd, sh)))
        assert all(torch.equal(outs[0][0], o[0]) and torch.equal(outs[0][1], o[1]) for o in outs)
        assert capi.status() == 0
        torch.save([t.cpu() for t in outs[0]], sys.argv[1])
    """)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    results = []
    for setting in ("0", "2", "7", "12"):
        path = os.path.join(root, "tests", f"_dyn_{setting}.pt")
        env = dict(os.environ, SPIO_DYN=setting, SPIO_DYN_MIN_PAIRS="8", PYTHONPATH=root)
        subprocess.run([sys.executable, "-c", code, path], check=True, env=env, cwd=root, timeout=300)
        results.append(torch.load(path))
        os.remove(path)
    for other in results[1:]:
        assert torch.equal(results[0][0], other[0]) and torch.equal(results[0][1], other[1])


def test_start_up_settings_give_identical_results():
    """SPIO_WARM (boxes requested from L2 before the kernel waits for its predecessors) and
    SPIO_PREFILL (stages requested before the load lane waits for the first one to land) change
    when data is asked for, never what is computed: fprop, dgrad and wgrad of a chain of dependent
    launches, in which each launch reads what the one before it wrote, must give the same bits with
    the requests and the window switched off, at their defaults, and at larger values."""
    import os
    import subprocess
    import sys
    import textwrap

    code = textwrap.dedent("""
        import sys, torch
        from oracle import oracle as O
        from tests import capi
        sh = O.Shape(24, 136, 30, 30, 3, 3, 1, 1)
        x, w, b, dy = O.make_inputs(sh, seed=33, bias=True)
        xd, wd, bd, dyd = (capi.to_dev(t) for t in (x, w, b, dy))
        ws = (wd.float() * 0.5).half().contiguous(memory_format=torch.channels_last)
        # Every launch consumes the output of the launch before it, and the launches follow each other
        # without anything in between (outputs are allocated first): a request that ran ahead of the
        # producer and were served stale data would show up here.
        import ctypes
        from spio_b200 import _clib
        lib = _clib.load()
        s = capi.cshape(sh); sp = ctypes.byref(s)
        st = torch.cuda.current_stream().cuda_stream
        mk = lambda: torch.full_like(xd, capi.DEAD_VALUE)
        y1, y2, y3, g1, g2 = mk(), mk(), mk(), mk(), mk()
        dw = torch.full((sh.c, 8, sh.r, sh.s), capi.DEAD_VALUE, dtype=torch.float32, device=xd.device).contiguous(memory_format=torch.channels_last)
        nbytes = lib.spio_conv2d_gw8_wgrad_scratch_bytes(sp, None)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device=xd.device)
        torch.cuda.synchronize()
        for src, dst in ((xd, y1), (y1, y2), (y2, y3)):
            _clib.check(lib.spio_conv2d_gw8_fprop(dst.data_ptr(), src.data_ptr(), ws.data_ptr(), bd.data_ptr(), sp, None, st))
        for src, dst in ((y3, g1), (g1, g2)):
            _clib.check(lib.spio_conv2d_gw8_dgrad(dst.data_ptr(), src.data_ptr(), ws.data_ptr(), sp, None, st))
        _clib.check(lib.spio_conv2d_gw8_wgrad(dw.data_ptr(), y2.data_ptr(), g2.data_ptr(), sp, None, scratch.data_ptr(), nbytes, st))
        torch.cuda.synchronize()
        # and the chain equals the same launches issued one by one with a synchronisation after each
        z1 = capi.fprop(xd, ws, bd, sh); torch.cuda.synchronize()
        z2 = capi.fprop(z1, ws, bd, sh); torch.cuda.synchronize()
        z3 = capi.fprop(z2, ws, bd, sh); torch.cuda.synchronize()
        h1 = capi.dgrad(z3, ws, sh); torch.cuda.synchronize()
        h2 = capi.dgrad(h1, ws, sh); torch.cuda.synchronize()
        assert torch.equal(y3, z3) and torch.equal(g2, h2)
        assert torch.equal(dw, capi.wgrad(z2, h2, sh))
        assert capi.status() == 0
        torch.save([t.cpu() for t in (y3, g2, dw)], sys.argv[1])
    """)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    results = []
    for warm, prefill in (("0", "0"), ("2", "2"), ("5", "1"), ("1", "3")):
        path = os.path.join(root, "tests", f"_warm_{warm}_{prefill}.pt")
        env = dict(os.environ, SPIO_WARM=warm, SPIO_PREFILL=prefill, PYTHONPATH=root)
        subprocess.run([sys.executable, "-c", code, path], check=True, env=env, cwd=root, timeout=300)
        results.append(torch.load(path))
        os.remove(path)
    for other in results[1:]:
        assert all(torch.equal(a, b) for a, b in zip(results[0], other))
    assert all(torch.isfinite(t.float()).all() for t in results[0])
