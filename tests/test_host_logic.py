"""Host-side pieces that need no GPU: layer matching, model transform, configuration spaces,
kernel cache overlay, parameter logging, tolerance helpers, performance-model choice."""

import pytest
import torch
from torch import nn

from spio_b200.cuda import B200_ATTRIBUTES
from spio_b200.kernels import (Conv2dGw8Config, Conv2dGw8Params, Conv2dGw8WgradConfig, KernelCache,
                               KernelKey, KernelParamsLogger, PerformanceModelCache,
                               conv2d_gw8_kernel_factory, conv2d_gw8_wgrad_kernel_factory)
from spio_b200.layers import Conv2dGw8, make_conv2d
from spio_b200.transform import scan_modules, transform
from spio_b200.transform._transform import _transform
from spio_b200.util import (assert_all_close_with_acc_depth, divup, next_relative_prime)


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.conv = nn.Conv2d(64, 64, 3, padding=1, groups=8)
        self.norm = nn.BatchNorm2d(64)
        self.pw = nn.Conv2d(64, 128, 1)
        self.tail = nn.Sequential(nn.Conv2d(128, 128, 5, padding=2, groups=16, bias=False), nn.ReLU())
        self.dw = nn.Conv2d(128, 128, 3, padding=1, groups=128)       # depthwise: not gw8
        self.strided = nn.Conv2d(128, 128, 3, stride=2, groups=16)    # stride 2: not gw8

    def forward(self, x):
        return self.strided(self.dw(self.tail(self.pw(self.norm(self.conv(x))))))


def test_match_args():
    assert Conv2dGw8.match_args(64, 64, 3, groups=8)
    assert Conv2dGw8.match_args(64, 64, (5, 1), groups=8)
    assert not Conv2dGw8.match_args(64, 128, 3, groups=8)
    assert not Conv2dGw8.match_args(64, 64, 3, groups=4)
    assert not Conv2dGw8.match_args(64, 64, 7, groups=8)
    assert not Conv2dGw8.match_args(64, 64, 3, stride=2, groups=8)
    assert not Conv2dGw8.match_args(64, 64, 3, dilation=2, groups=8)
    assert not Conv2dGw8.match_args(64, 64, 3, groups=8, padding_mode="reflect")
    assert isinstance(make_conv2d(64, 64, 3, groups=8), Conv2dGw8)
    assert make_conv2d(64, 64, 3, groups=2) is None


def test_transform_replaces_exactly_the_matching_modules():
    model = Block()
    traced, n = _transform(model)
    assert n == 2
    assert isinstance(traced.conv, Conv2dGw8) and isinstance(traced.tail.get_submodule("0"), Conv2dGw8)
    assert not isinstance(traced.dw, Conv2dGw8) and not isinstance(traced.strided, Conv2dGw8)
    assert traced.conv.weight is model.conv.weight and traced.conv.bias is model.conv.bias
    assert sorted(traced.state_dict()) == sorted(model.state_dict())
    assert isinstance(transform(Block()), torch.fx.GraphModule)
    again, n2 = _transform(traced)
    assert n2 == 0
    with pytest.raises(ValueError):
        Conv2dGw8.from_torch_module(model.dw)


def test_scan_modules():
    got = scan_modules(Block(), torch.randn(2, 64, 12, 10))
    assert got == [Conv2dGw8Params(n=2, c=64, h=12, w=10, padding=(1, 1), has_bias=True),
                   Conv2dGw8Params(n=2, c=128, h=12, w=10, padding=(2, 2), r=5, s=5)]


def test_operator_rejects_cpu_tensors_and_bad_arguments():
    from spio_b200.functional import conv2d_gw8

    x = torch.randn(1, 16, 8, 8).half()
    w = torch.randn(16, 8, 3, 3).half()
    with pytest.raises(ValueError, match="CUDA devices only"):
        conv2d_gw8(x, w, None, 1, 1, 1, 1, 2)
    with pytest.raises(AssertionError):
        conv2d_gw8(x.float(), w, None, 1, 1, 1, 1, 2)
    with pytest.raises(AssertionError):
        conv2d_gw8(x, w, None, 2, 1, 1, 1, 2)
    with pytest.raises(AssertionError):
        conv2d_gw8(x, w, None, 1, 1, 1, 1, 1)


def test_fake_implementations_give_shapes_without_a_device():
    x = torch.empty(2, 32, 9, 7, dtype=torch.float16, device="meta")
    w = torch.empty(32, 8, 3, 3, dtype=torch.float16, device="meta")
    y = torch.ops.spio.conv2d_gw8(x, w, None, 1, 1, 1, 1, 4)
    assert tuple(y.shape) == (2, 32, 9, 7) and y.dtype == torch.float16
    assert y.is_contiguous(memory_format=torch.channels_last)
    gi, gw, gb = torch.ops.spio.conv2d_gw8_backward(x, w, None, y, 1, 1, True, True, False)
    assert tuple(gi.shape) == (2, 32, 9, 7) and gw.dtype == torch.float32 and gb.numel() == 0


def test_configuration_spaces():
    p = Conv2dGw8Params(n=128, c=64, h=56, w=56)
    fwd = list(conv2d_gw8_kernel_factory.configs(p, B200_ATTRIBUTES))
    bwd = list(conv2d_gw8_kernel_factory.configs(p, B200_ATTRIBUTES, igrad=True))
    wg = list(conv2d_gw8_wgrad_kernel_factory.configs(p, B200_ATTRIBUTES))
    assert len(fwd) > 20 and len(fwd) == len(set(fwd)) and len(bwd) == len(fwd)
    assert all(isinstance(c, Conv2dGw8Config) for c in fwd)
    assert all(isinstance(c, Conv2dGw8WgradConfig) for c in wg) and len(wg) > 10
    assert all(c.nb * c.ncb <= c.wpg * c.tpw for c in wg)
    assert all(c.nb * ((c.ncb + 1) // 2) <= c.wpg * ((c.tpw + 1) // 2) for c in fwd)
    tall = Conv2dGw8Params(n=4, c=32, h=20, w=20, padding=2, r=5, s=5)
    assert all(c.tpw <= 2 for c in conv2d_gw8_kernel_factory.configs(tall, B200_ATTRIBUTES))


def test_kernel_names_and_compile_without_device():
    p = Conv2dGw8Params(n=4, c=64, h=16, w=32, has_bias=True)
    f = conv2d_gw8_kernel_factory
    assert f.get_kernel_name() == "spio_conv2d_gw8_fprop"
    assert f.get_kernel_name(igrad=True) == "spio_conv2d_gw8_dgrad"
    assert f.get_full_kernel_name(p) == "spio_conv2d_gw8_fprop__4n_64c_16h_32w_1py_1px_3r_3s_b"
    assert conv2d_gw8_wgrad_kernel_factory.get_kernel_name() == "spio_conv2d_gw8_wgrad"
    k = f.make_kernel(p, Conv2dGw8Config(wpg=2, tpw=2, pps=1), B200_ATTRIBUTES)
    k.compile(B200_ATTRIBUTES)
    assert k.plan["wpg"] == 2 and k.plan["tpw"] == 2 and k.launch_params.block == 640
    bad = f.make_kernel(p, Conv2dGw8Config(wpg=5), B200_ATTRIBUTES)
    with pytest.raises(ValueError, match="variant"):
        bad.compile(B200_ATTRIBUTES)
    with pytest.raises(ValueError, match="not loaded"):
        k.launch(None, None, None, None)
    assert f.get_kernel_cache() is f.get_kernel_cache()
    assert f.get_kernel_cache() is not f.get_kernel_cache(igrad=True)


def test_kernel_cache_overlay():
    p = Conv2dGw8Params(n=4, c=64, h=16, w=32)
    other = Conv2dGw8Params(n=8, c=64, h=16, w=32)
    cache = KernelCache()
    k = conv2d_gw8_kernel_factory.make_kernel(p, Conv2dGw8Config(), B200_ATTRIBUTES)
    cache.update_overlay({KernelKey(device_ordinal=0, params=p): k})
    assert cache.get(conv2d_gw8_kernel_factory, p, torch.device("cuda", 0)) is k
    with pytest.raises(ValueError, match="not found in overlay cache"):
        cache.get(conv2d_gw8_kernel_factory, other, torch.device("cuda", 0))
    with KernelParamsLogger() as logger:
        cache.get(conv2d_gw8_kernel_factory, p, torch.device("cuda", 0))
        cache.get(conv2d_gw8_kernel_factory, p, torch.device("cuda", 0))
    logged = logger.get_logged_params()
    assert len(logged) == 1 and logged[0][1] == p
    cache.clear_overlay()
    cache.clear_cache()


def test_performance_model_table_round_trip(tmp_path, monkeypatch):
    monkeypatch.setenv("SPIO_CACHE_DIR", str(tmp_path))
    pm = PerformanceModelCache()
    p = Conv2dGw8Params(n=128, c=64, h=56, w=56)
    cfg = Conv2dGw8Config(wpg=2, tpw=4, pps=1, ncb=7, nb=1, ns=8, nob=3)
    path = pm.record("spio_conv2d_gw8_fprop", "sm_100a", p, cfg)
    assert path.parent == tmp_path
    assert pm._table("spio_conv2d_gw8_fprop", "sm_100a")[p.encode()] == cfg.as_tune()


def test_gbt_model_json_round_trip():
    from spio_b200.kernels.gbt_model import GbtModel

    rows = [{"n": float(n), "ns": float(ns)} for n in (1, 8, 64, 512) for ns in (3, 6, 12)]
    target = [r["n"] * 0.1 + (12 - r["ns"]) * 0.5 for r in rows]
    model = GbtModel.fit(rows, target, n_trees=60, depth=3, learning_rate=0.3)
    again = GbtModel.from_json(model.to_json())
    pred = again.predict(rows)
    assert pred == model.predict(rows)
    assert max(abs(a - b) for a, b in zip(pred, target)) < 0.15 * max(target)


def test_util_helpers():
    assert divup(7, 2) == 4 and divup(8, 2) == 4
    assert next_relative_prime(8, 8) == 9 and next_relative_prime(9, 8) == 9
    a = torch.ones(4)
    assert_all_close_with_acc_depth(a, a + 1e-5, acc_depth=72)
    with pytest.raises(AssertionError, match="Tensors not close"):
        assert_all_close_with_acc_depth(a, a + 1.0, acc_depth=72, msg="ctx")


def test_layernorm_2d_layer_and_op_checks():
    """Host-side behaviour of LayerNorm2d that needs no GPU."""
    import torch
    from torch import nn

    from spio_b200.functional import layernorm_2d
    from spio_b200.layers import LayerNorm2d

    ln = LayerNorm2d(96, eps=1e-5)
    assert ln.weight.shape == (96,) and ln.bias.dtype == torch.float32 and "96" in repr(ln)
    assert LayerNorm2d(64, elementwise_affine=False).weight is None
    assert LayerNorm2d.match(nn.LayerNorm(192)) and not LayerNorm2d.match(nn.LayerNorm(100))
    assert not LayerNorm2d.match(nn.LayerNorm((4, 8))) and not LayerNorm2d.match(nn.BatchNorm2d(64))
    src = nn.LayerNorm(384, eps=1e-6)
    assert LayerNorm2d.from_torch_module(src).weight is src.weight
    with pytest.raises(ValueError):
        LayerNorm2d(12)
    with pytest.raises(Exception, match="CUDA"):
        layernorm_2d(torch.zeros(1, 64, 2, 2, dtype=torch.float16))
    # fake (meta) implementation: shapes and dtypes without a device
    y, stats = torch.ops.spio.layernorm_2d(torch.empty(2, 64, 3, 5, dtype=torch.float16, device="meta"), None, None, 1e-6)
    assert y.shape == (2, 64, 3, 5) and stats.shape == (30, 2) and stats.dtype == torch.float32


def test_every_plannable_shape_has_a_configuration():
    """A wide image with a large filter needs more column tiles than the enumeration tries;
    the planner's own choice is always part of the configuration space."""
    from spio_b200.cuda import B200_ATTRIBUTES
    from spio_b200.kernels import (Conv2dGw8Params, conv2d_gw8_kernel_factory,
                                   conv2d_gw8_wgrad_kernel_factory)

    for p in (Conv2dGw8Params(n=32, c=64, h=112, w=112, r=5, s=5, padding=2),
              Conv2dGw8Params(n=2, c=8, h=9, w=300, r=3, s=3, padding=1),
              Conv2dGw8Params(n=1, c=1024, h=3, w=3, r=1, s=1, padding=0)):
        assert len(list(conv2d_gw8_kernel_factory.configs(p, B200_ATTRIBUTES))) > 0
        assert len(list(conv2d_gw8_kernel_factory.configs(p, B200_ATTRIBUTES, igrad=True))) > 0
        assert len(list(conv2d_gw8_wgrad_kernel_factory.configs(p, B200_ATTRIBUTES))) > 0


def test_table_entries_are_capped_to_the_196_kib_configuration():
    """A tuned entry that asks for a ring above the soft shared-memory cap hands the depth back
    to the planner; entries within the cap, and tcgen05 entries, are left alone."""
    from spio_b200.kernels import conv2d_gw8_kernel_factory as factory
    from spio_b200.kernels.conv2d_gw8_kernel import SMEM_SOFT_CAP, plan_is_valid
    from spio_b200 import _clib

    params = Conv2dGw8Params(n=256, c=64, h=56, w=56, r=3, s=3, padding=1)
    deep = Conv2dGw8Config(wpg=2, tpw=4, pps=2, ns=5, nob=2)
    assert plan_is_valid(_clib.FPROP, params, deep.as_tune(), B200_ATTRIBUTES)
    assert not plan_is_valid(_clib.FPROP, params, deep.as_tune(), B200_ATTRIBUTES, SMEM_SOFT_CAP)
    fixed = factory.fixup_config(params, deep, B200_ATTRIBUTES)
    assert fixed.ns == 0 and (fixed.wpg, fixed.tpw, fixed.pps, fixed.nob) == (2, 4, 2, 2)
    assert plan_is_valid(_clib.FPROP, params, fixed.as_tune(), B200_ATTRIBUTES, SMEM_SOFT_CAP)
    ok = Conv2dGw8Config(wpg=2, tpw=4, pps=2, ns=4, nob=2)
    assert factory.fixup_config(params, ok, B200_ATTRIBUTES, igrad=True) == ok
    tc = Conv2dGw8Config(engine=2, ns=6, nob=2)
    assert factory.fixup_config(params, tc, B200_ATTRIBUTES) == tc
