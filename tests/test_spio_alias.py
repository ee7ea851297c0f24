"""The reference's import name: ``import spio`` and its subpackages resolve to this package's modules
(the same module objects, so the operators are registered once)."""

import importlib


def test_spio_names_resolve_to_spio_b200_modules():
    import spio
    import spio_b200
    from spio.functional import conv2d_gw8
    from spio.kernels import (Conv2dGw8Config, Conv2dGw8Params, Conv2dGw8WgradConfig, KernelFactory, Stats,
                              conv2d_gw8_kernel_factory, conv2d_gw8_wgrad_kernel_factory)
    from spio.layers import Conv2dGw8, make_conv2d
    from spio.transform import scan_modules, transform
    import spio.compiler
    import spio.cuda.driver
    import spio.generators
    import spio.util

    assert spio.__version__ == spio_b200.__version__
    import spio_b200.functional
    import spio_b200.kernels.conv2d_gw8_params as real

    assert conv2d_gw8 is spio_b200.functional.conv2d_gw8
    assert importlib.import_module("spio.kernels.conv2d_gw8_params") is real
    assert Conv2dGw8Params is real.Conv2dGw8Params
    assert spio.kernels is spio_b200.kernels and spio.layers.Conv2dGw8 is Conv2dGw8
    assert callable(transform) and callable(scan_modules) and callable(make_conv2d)
    assert spio.util.divup(7, 2) == 4
    assert all(x is not None for x in (Conv2dGw8Config, Conv2dGw8WgradConfig, KernelFactory, Stats,
                                       conv2d_gw8_kernel_factory, conv2d_gw8_wgrad_kernel_factory))
    assert spio.generators.Generators is not None and spio.compiler.compile_kernel is not None


def test_unknown_names_fail_normally():
    import pytest

    import spio

    with pytest.raises(ImportError):
        importlib.import_module("spio.no_such_module")
    with pytest.raises(AttributeError):
        spio.no_such_attribute
