"""``spio``: the reference's import name for this package.

Code written for andravin/spio imports ``spio.functional``, ``spio.layers``, ``spio.transform``,
``spio.kernels``, ``spio.compiler``, ``spio.cuda``, ``spio.util`` and ``spio.generators``
(reference: spio/__init__.py:1-22 and the ``__init__`` of each subpackage).  Every such name
resolves to the module of the same name in :mod:`spio_b200` -- the SAME module object, so the
``spio::conv2d_gw8`` operators are registered once however the package is imported.

Like ``spio_b200`` (and unlike the reference, which initialises the CUDA driver at import),
importing this package loads neither torch nor the native library.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.machinery
import sys

import spio_b200 as _impl

__version__ = _impl.__version__
supported_arch = _impl.supported_arch

_REAL = "spio_b200"


class _AliasLoader(importlib.abc.Loader):
    """Hands out the already imported ``spio_b200.<x>`` module under the name ``spio.<x>``."""

    def __init__(self, real_name: str):
        self._real_name = real_name

    def create_module(self, spec):
        module = importlib.import_module(self._real_name)
        self._identity = (module.__spec__, getattr(module, "__loader__", None))
        return module

    def exec_module(self, module):
        # The real module has been executed; re-running it would register the operators twice.
        # The import system has just stamped the alias spec on it: put its own back.
        module.__spec__, module.__loader__ = self._identity


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if not fullname.startswith(__name__ + "."):
            return None
        real_name = _REAL + fullname[len(__name__):]
        try:
            real_spec = importlib.util.find_spec(real_name)
        except (ImportError, ValueError):
            return None
        if real_spec is None:
            return None
        spec = importlib.machinery.ModuleSpec(fullname, _AliasLoader(real_name),
                                              is_package=real_spec.submodule_search_locations is not None)
        return spec


import importlib.util  # noqa: E402  (used by the finder)

if not any(isinstance(f, _AliasFinder) for f in sys.meta_path):
    sys.meta_path.insert(0, _AliasFinder())


def __getattr__(name: str):
    """``spio.kernels`` etc. without an explicit ``import spio.kernels``."""
    try:
        return importlib.import_module(f"{__name__}.{name}")
    except ImportError as exc:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from exc
