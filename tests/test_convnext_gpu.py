"""One train step of the ConvNeXt-T-style network (3x3 gw8 convolutions, widths 96/192/384/768,
depths 3/3/9/3) before and after ``transform``: 18 layers are swapped and loss and gradients
agree with the cuDNN path within fp16 tolerance."""

import pytest
import torch

from spio_b200.examples.convnext_gw8 import ConvNeXtGw8, train_step
from spio_b200.kernels import device_status
from spio_b200.layers import Conv2dGw8
from spio_b200.transform import scan_modules
from spio_b200.transform._transform import _transform

@pytest.mark.gpu
def test_convnext_train_step_matches_cudnn():
    torch.manual_seed(1234 + 4)
    dev = torch.device("cuda")
    model = ConvNeXtGw8().to(dev).to(memory_format=torch.channels_last)
    images = torch.randn(8, 3, 224, 224, device=dev).contiguous(memory_format=torch.channels_last)
    labels = torch.randint(0, 1000, (8,), device=dev)

    ref_loss = train_step(model, images, labels)
    ref_grads = {n: p.grad.clone() for n, p in model.named_parameters()}
    model.zero_grad(set_to_none=True)

    fast, replaced = _transform(model)
    assert replaced == 18
    assert sum(isinstance(m, Conv2dGw8) for m in fast.modules()) == 18
    loss = train_step(fast, images, labels)
    assert device_status() == 0
    assert abs(float(loss) - float(ref_loss)) <= 2e-2 * abs(float(ref_loss))
    checked = 0
    for name, p in fast.named_parameters():
        if name.endswith("conv.weight"):
            g, r = p.grad.float(), ref_grads[name].float()
            assert float((g - r).abs().max()) <= 5e-2 * float(r.abs().max()) + 1e-6, name
            checked += 1
    assert checked == 18


def test_scan_modules_lists_the_gw8_layers():
    model = ConvNeXtGw8(depths=(1, 1, 1, 1))
    shapes = scan_modules(model, torch.randn(2, 3, 64, 64))
    assert [(p.c, p.h) for p in shapes] == [(96, 16), (192, 8), (384, 4), (768, 2)]
    assert all(p.r == 3 and p.has_bias for p in shapes)


@pytest.mark.gpu
def test_convnext_train_step_with_fused_layernorm():
    """Swapping the channel LayerNorms for spio_b200.layers.LayerNorm2d keeps loss and
    gradients of the train step within fp16 tolerance of the torch LayerNorm path."""
    from spio_b200.examples.convnext_gw8 import swap_layernorm
    from spio_b200.layers import LayerNorm2d

    torch.manual_seed(1234 + 4)
    dev = torch.device("cuda")
    model = ConvNeXtGw8().to(dev).to(memory_format=torch.channels_last)
    images = torch.randn(8, 3, 224, 224, device=dev).contiguous(memory_format=torch.channels_last)
    labels = torch.randint(0, 1000, (8,), device=dev)
    fast, _ = _transform(model)
    ref_loss = train_step(fast, images, labels)
    ref_grads = {id(p): p.grad.clone() for p in fast.parameters()}   # parameters are shared, not copied
    fast.zero_grad(set_to_none=True)

    swapped = swap_layernorm(model)
    assert swapped == 22  # stem + 3 downsampling + 18 blocks
    fused, replaced = _transform(model)
    assert replaced == 18
    assert sum(isinstance(m, LayerNorm2d) for m in model.modules()) == 22
    # tracing looks through the layer, so the transformed graph calls the operator directly
    assert sum("layernorm_2d" in str(n.target) for n in fused.graph.nodes if n.op == "call_function") == 22
    loss = train_step(fused, images, labels)
    assert device_status() == 0
    assert abs(float(loss) - float(ref_loss)) <= 2e-2 * abs(float(ref_loss))
    worst, checked = 0.0, 0
    for p in fused.parameters():
        r = ref_grads[id(p)].float()
        worst = max(worst, float((p.grad.float() - r).abs().max()) / (float(r.abs().max()) + 1e-12))
        checked += 1
    assert checked == len(ref_grads) and worst <= 8e-2, worst
