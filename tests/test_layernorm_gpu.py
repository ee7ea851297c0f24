"""LayerNorm2d (spio::layernorm_2d) against torch's CPU layer_norm in float64: forward,
backward (input, weight and bias gradients), reproducibility, autocast, module swap."""

import pytest
import torch
from torch import nn

from spio_b200.functional import layernorm_2d, layernorm_2d_op
from spio_b200.layers import LayerNorm2d

pytestmark = pytest.mark.gpu

CL = torch.channels_last
SHAPES = [(2, 64, 5, 7), (3, 96, 14, 14), (2, 192, 9, 9), (1, 384, 7, 5), (2, 768, 3, 3), (1, 1024, 4, 4),
          (4, 8, 6, 6), (2, 200, 5, 5), (1, 40, 33, 3), (64, 96, 56, 56)]


def reference(x, w, b, eps, dy=None):
    """float64 CPU LayerNorm over the channels; gradients through autograd."""
    xr = x.detach().double().cpu().permute(0, 2, 3, 1).requires_grad_(True)
    wr = w.detach().double().cpu().requires_grad_(True) if w is not None else None
    br = b.detach().double().cpu().requires_grad_(True) if b is not None else None
    y = torch.nn.functional.layer_norm(xr, (x.shape[1],), wr, br, eps)
    out = [y.permute(0, 3, 1, 2)]
    if dy is not None:
        y.backward(dy.detach().double().cpu().permute(0, 2, 3, 1))
        out += [xr.grad.permute(0, 3, 1, 2), wr.grad if wr is not None else None, br.grad if br is not None else None]
    return out


def make(shape, affine=True, seed=0):
    g = torch.Generator().manual_seed(seed)
    n, c, h, w = shape
    x = (torch.randn(shape, generator=g) * 1.5 + 0.3).half().cuda().contiguous(memory_format=CL)
    dy = torch.randn(shape, generator=g).half().cuda().contiguous(memory_format=CL)
    wt = (1 + 0.2 * torch.randn(c, generator=g)).cuda() if affine else None
    bs = (0.1 * torch.randn(c, generator=g)).cuda() if affine else None
    return x, dy, wt, bs


@pytest.mark.parametrize("shape", SHAPES, ids=str)
@pytest.mark.parametrize("affine", [True, False])
def test_forward(shape, affine):
    x, _, w, b = make(shape, affine)
    y, stats = layernorm_2d_op(x, w, b, 1e-6)
    (ref,) = reference(x, w, b, 1e-6)
    assert y.is_contiguous(memory_format=CL) and y.dtype == torch.float16
    err = (y.double().cpu() - ref).abs().max().item()
    assert err <= 2e-3 * ref.abs().max().item() + 1e-3, err
    xr = x.double().cpu().permute(0, 2, 3, 1).reshape(-1, shape[1])
    torch.testing.assert_close(stats[:, 0].double().cpu(), xr.mean(1), rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(stats[:, 1].double().cpu(), (xr.var(1, unbiased=False) + 1e-6).rsqrt(), rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("shape", SHAPES, ids=str)
def test_backward(shape):
    x, dy, w, b = make(shape, True, seed=3)
    x.requires_grad_(True), w.requires_grad_(True), b.requires_grad_(True)
    y = layernorm_2d(x, w, b, 1e-6)
    y.backward(dy)
    _, dx_ref, dw_ref, db_ref = reference(x, w, b, 1e-6, dy)
    assert (x.grad.double().cpu() - dx_ref).abs().max().item() <= 2e-3 * dx_ref.abs().max().item() + 1e-3
    rows = shape[0] * shape[2] * shape[3]
    tol = 2e-3 * rows ** 0.5 + 1e-2   # fp16 data, fp32 sums over `rows` pixels
    assert (w.grad.double().cpu() - dw_ref).abs().max().item() <= tol
    assert (b.grad.double().cpu() - db_ref).abs().max().item() <= tol
    assert w.grad.dtype == torch.float32 and x.grad.dtype == torch.float16


def test_backward_is_reproducible_and_input_grad_only():
    x, dy, w, b = make((8, 192, 28, 28), True, seed=5)
    grads = []
    for _ in range(2):
        xx, ww, bb = x.clone().requires_grad_(True), w.clone().requires_grad_(True), b.clone().requires_grad_(True)
        layernorm_2d(xx, ww, bb).backward(dy)
        grads.append((xx.grad, ww.grad, bb.grad))
    for a, c in zip(*grads):
        assert torch.equal(a, c)
    xx = x.clone().requires_grad_(True)
    layernorm_2d(xx, w, b).backward(dy)     # weight and bias do not require grad
    assert torch.equal(xx.grad, grads[0][0])


def test_module_matches_permuted_torch_layernorm_under_autocast():
    torch.manual_seed(0)
    ref = nn.LayerNorm(96, eps=1e-6).cuda()
    with torch.no_grad():
        ref.weight.uniform_(0.5, 1.5), ref.bias.uniform_(-0.2, 0.2)
    assert LayerNorm2d.match(ref)
    fused = LayerNorm2d.from_torch_module(ref)
    assert fused.weight is ref.weight
    x = torch.randn(4, 96, 20, 20, device="cuda").contiguous(memory_format=CL).requires_grad_(True)
    x2 = x.detach().clone().requires_grad_(True)
    with torch.autocast("cuda", dtype=torch.float16):
        y = fused(x)
        y_ref = ref(x2.permute(0, 2, 3, 1)).permute(0, 3, 1, 2)
    assert y.dtype == x.dtype  # the autocast rule returns the input's dtype
    torch.testing.assert_close(y.float(), y_ref.float(), rtol=2e-3, atol=4e-3)
    dy = torch.randn_like(y)
    y.backward(dy)
    gw = ref.weight.grad.clone()
    ref.weight.grad = None
    y_ref.backward(dy)
    torch.testing.assert_close(x.grad, x2.grad, rtol=5e-3, atol=5e-3)
    torch.testing.assert_close(gw, ref.weight.grad, rtol=5e-3, atol=5e-2)


def test_rejects_what_it_cannot_do():
    with pytest.raises(ValueError):
        LayerNorm2d(100)
    with pytest.raises(ValueError):
        LayerNorm2d(2048)
    with pytest.raises(Exception):
        layernorm_2d(torch.randn(1, 64, 4, 4).half())   # CPU tensor
    with pytest.raises(Exception):
        layernorm_2d(torch.randn(1, 64, 4, 4, device="cuda"))   # fp32 outside autocast
