"""The PyTorch operator, its autograd formula, the layer and the model transform on a GPU
(reference: tests/test_conv2d_gw8.py:176-236 via spio/src_tests/run_test.py:128-246)."""

import pytest
import torch
from torch import nn

from oracle import oracle as O
from spio_b200.functional import conv2d_gw8
from spio_b200.kernels import KernelParamsLogger, device_status
from spio_b200.layers import Conv2dGw8
from spio_b200.transform._transform import _transform
from tests.shapes import REFERENCE_TEST_SHAPES, ident

pytestmark = pytest.mark.gpu
CL = torch.channels_last


def _dev(t):
    return None if t is None else (t.cuda().contiguous(memory_format=CL) if t.dim() == 4 else t.cuda())


@pytest.mark.parametrize("case", REFERENCE_TEST_SHAPES[::4], ids=ident)
def test_function_and_gradients(case):
    sh, has_bias = case
    x, w, b, dy = O.make_inputs(sh, seed=21, bias=has_bias)
    xd, wd, bd = _dev(x).requires_grad_(True), _dev(w).requires_grad_(True), _dev(b)
    if bd is not None:
        bd.requires_grad_(True)
    y = conv2d_gw8(xd, wd, bd, stride=1, padding_y=sh.pad_h, padding_x=sh.pad_w, groups=sh.groups)
    assert y.is_contiguous(memory_format=CL) and y.dtype == torch.float16
    wanted = (xd, wd) + ((bd,) if has_bias else ())
    grads = torch.autograd.grad(y, wanted, _dev(dy))
    assert device_status() == 0
    O.assert_close(y, O.torch_fprop(x, w, b, sh), sh, "fprop", ident(case))
    dx, dw = O.torch_grads(x, w, dy, sh)
    O.assert_close(grads[0], dx, sh, "dgrad", ident(case))
    # autograd hands the fp32 kernel result back in the weight's dtype (fp16 here)
    O.assert_close(grads[1], dw, sh, "wgrad", ident(case), atol_scale=1.0 + 1e-3 * float(dw.abs().max())
                   / O.reference_tolerance(sh, "wgrad")[0])
    if has_bias:
        assert torch.allclose(grads[2].cpu(), dy.float().sum(dim=(0, 2, 3)), rtol=2e-3, atol=2e-2)


def test_nchw_strided_inputs_are_accepted():
    sh = O.Shape(2, 32, 10, 12, 3, 3, 1, 1)
    x, w, _, _ = O.make_inputs(sh, seed=22, bias=False)
    y = conv2d_gw8(x.cuda(), w.cuda(), None, 1, 1, 1, 1, sh.groups)     # plain contiguous NCHW
    O.assert_close(y, O.torch_fprop(x, w, None, sh), sh, "fprop", "nchw")


def test_only_requested_gradients_are_computed():
    sh = O.Shape(2, 16, 8, 8, 3, 3, 1, 1)
    x, w, _, dy = O.make_inputs(sh, seed=23, bias=False)
    gi, gw, gb = torch.ops.spio.conv2d_gw8_backward(_dev(x), _dev(w), None, _dev(dy), 1, 1, True, False, False)
    assert gi.numel() == x.numel() and gw.numel() == 0 and gb.numel() == 0
    xd = _dev(x).requires_grad_(True)
    y = conv2d_gw8(xd, _dev(w), None, 1, 1, 1, 1, sh.groups)
    (dx,) = torch.autograd.grad(y, (xd,), _dev(dy))
    O.assert_close(dx, O.torch_grads(x, w, dy, sh)[0], sh, "dgrad", "input grad only")


class Net(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.conv = nn.Conv2d(c, c, 3, padding=1, groups=c // 8)
        self.act = nn.GELU()
        self.pw = nn.Conv2d(c, c, 1)

    def forward(self, x):
        return self.pw(self.act(self.conv(x)))


@pytest.mark.parametrize("c,hw", [(64, 28), (96, 14)])
def test_layer_through_transform_under_autocast(c, hw):
    torch.manual_seed(0)
    model = Net(c).cuda().to(memory_format=CL)
    x = torch.randn(4, c, hw, hw, device="cuda").contiguous(memory_format=CL)
    with torch.autocast("cuda", dtype=torch.float16):
        ref = model(x)
    ref.float().square().mean().backward()
    ref_grad = model.conv.weight.grad.clone()
    model.zero_grad()
    fast, n = _transform(model)
    assert n == 1 and isinstance(fast.conv, Conv2dGw8)
    with KernelParamsLogger() as logger, torch.autocast("cuda", dtype=torch.float16):
        out = fast(x)
    assert len(logger.get_logged_params()) == 1
    out.float().square().mean().backward()
    assert device_status() == 0
    assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
    got = fast.conv.weight.grad
    assert got.dtype == torch.float32
    assert float((got - ref_grad).abs().max()) <= 2e-2 * float(ref_grad.abs().max()) + 1e-6


def test_opcheck():
    sh = O.Shape(4, 64, 16, 32, 3, 3, 1, 1)
    x, w, b, _ = O.make_inputs(sh, seed=24, bias=True)
    args = (_dev(x).requires_grad_(True), _dev(w).requires_grad_(True), _dev(b).requires_grad_(True))
    kwargs = dict(stride=1, padding_y=1, padding_x=1, dilation=1, groups=sh.groups)
    torch.library.opcheck(torch.ops.spio.conv2d_gw8.default, args, kwargs,
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


def test_layer_under_torch_compile():
    """The layer inside a torch.compile'd module (the operator is opaque to the compiler; its
    fake implementations and autograd registration must hold up) gives the eager results.
    Mirrors the reference's tests/test_conv2d_gw8.py:227-230."""
    torch.manual_seed(1)
    model = Net(64).cuda().to(memory_format=CL)
    fast, n = _transform(model)
    assert n == 1
    x = torch.randn(4, 64, 24, 24, device="cuda").contiguous(memory_format=CL)
    with torch.autocast("cuda", dtype=torch.float16):
        eager = fast(x)
    eager.float().square().mean().backward()
    eager_grad = fast.conv.weight.grad.clone()
    fast.zero_grad()
    compiled = torch.compile(fast)
    with torch.autocast("cuda", dtype=torch.float16):
        out = compiled(x)
    out.float().square().mean().backward()
    assert device_status() == 0
    assert torch.allclose(out.float(), eager.float(), rtol=1e-2, atol=1e-2)
    got = fast.conv.weight.grad
    assert float((got - eager_grad).abs().max()) <= 1e-2 * float(eager_grad.abs().max()) + 1e-6


def test_layernorm_opcheck():
    from spio_b200.functional import layernorm_2d  # noqa: F401  (registers the operator)

    x = torch.randn(2, 64, 5, 6, device="cuda").half().contiguous(memory_format=CL).requires_grad_(True)
    w = torch.rand(64, device="cuda").requires_grad_(True)
    b = torch.rand(64, device="cuda").requires_grad_(True)
    torch.library.opcheck(torch.ops.spio.layernorm_2d.default, (x, w, b, 1e-6),
                          test_utils=("test_schema", "test_faketensor", "test_autograd_registration"))


def test_operator_step_replayed_from_a_cuda_graph():
    """Forward and autograd of the operator captured with torch.cuda.graph and replayed on new
    data give the eager results bit for bit.  The operator costs the host a few hundred
    microseconds per step (torch's custom-operator and autograd machinery), more than its kernels
    take on small layers; a captured step has no host cost, so it must be capturable: the
    kernels' launches are recorded with their programmatic-launch attributes, the scratch buffer
    of the capturing stream comes from the graph's pool, and recorded forward launches split their
    work statically."""
    n, c, hw = 16, 72, 28
    gen = torch.Generator(device="cuda").manual_seed(5)
    mk = lambda *shape: torch.randn(*shape, device="cuda", generator=gen)  # noqa: E731
    w = (mk(c, 8, 3, 3) / 72 ** 0.5).half().contiguous(memory_format=CL).requires_grad_(True)
    bias = mk(c).requires_grad_(True)
    data = [(mk(n, c, hw, hw).half().contiguous(memory_format=CL), mk(n, c, hw, hw).half().contiguous(memory_format=CL))
            for _ in range(3)]

    def step(x, dy, w, bias):
        y = conv2d_gw8(x, w, bias, 1, 1, 1, 1, c // 8)
        return (y,) + torch.autograd.grad(y, (x, w, bias), dy)

    eager = [step(x.clone().requires_grad_(True), dy, w, bias) for x, dy in data]
    torch.cuda.synchronize()

    # The captured step gets leaf tensors of its own, first used on the capturing stream: autograd ties a
    # leaf to the stream it was first used on and synchronises with that stream in every backward pass,
    # which a capture does not survive if it is another stream.
    w, bias = w.detach().clone().requires_grad_(True), bias.detach().clone().requires_grad_(True)
    static_x = data[0][0].clone().requires_grad_(True)
    static_dy = data[0][1].clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):   # warm-up on the capturing stream, as torch asks for before a capture
            step(static_x, static_dy, w, bias)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        outs = step(static_x, static_dy, w, bias)
    for (x, dy), ref in zip(data, eager):
        with torch.no_grad():
            static_x.copy_(x)
            static_dy.copy_(dy)
        graph.replay()
        torch.cuda.synchronize()
        for got, want in zip(outs, ref):
            assert torch.equal(got, want)
    assert device_status() == 0
