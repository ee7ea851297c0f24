"""Swap supported ``nn.Conv2d`` modules of a model for this package's layers.

``transform`` and ``scan_modules`` behave like the reference's
(spio/transform/_transform.py:16-108): the model is traced with torch.fx, every
``call_module`` node whose module a layer class matches is served by a new layer that
shares the old parameters, and a ``GraphModule`` is returned.  Because the replacement
keeps the submodule's qualified name, the graph itself needs no rewriting: the module is
replaced under its parent and the graph recompiled.
"""

from __future__ import annotations

from typing import List, Tuple

import torch
from torch import fx

from ..layers import Conv2dGw8
from ..util.logger import log

spio_modules_classes = [Conv2dGw8]


def _matching_class(module):
    for cls in spio_modules_classes:
        if cls.match(module):
            return cls
    return None


def _set_submodule(root: torch.nn.Module, qualified_name: str, new: torch.nn.Module) -> None:
    parent_name, _, leaf = qualified_name.rpartition(".")
    parent = root.get_submodule(parent_name) if parent_name else root
    setattr(parent, leaf, new)


def _transform(model: torch.nn.Module) -> Tuple[fx.GraphModule, int]:
    """The transformed model and how many modules were replaced."""
    traced = fx.symbolic_trace(model)
    replaced = 0
    done = set()
    for node in traced.graph.nodes:
        if node.op != "call_module" or node.target in done:
            continue
        module = traced.get_submodule(node.target)
        cls = _matching_class(module)
        if cls is None:
            continue
        new = cls.from_torch_module(module)
        _set_submodule(traced, node.target, new)
        done.add(node.target)
        replaced += 1
        log(f"replaced a {type(module).__module__}.{type(module).__qualname__} module with "
            f"{type(new).__module__}.{new}")
    traced.delete_all_unused_submodules()
    traced.recompile()
    return traced, replaced


def transform(model: torch.nn.Module) -> fx.GraphModule:
    """The model with every supported module replaced by its counterpart of this package."""
    return _transform(model)[0]


class _ScanInterpreter(fx.Interpreter):
    def __init__(self, graph_module: fx.GraphModule):
        super().__init__(graph_module)
        self.params_lst: List = []

    def call_module(self, target, args, kwargs):
        module = self.fetch_attr(target)
        cls = _matching_class(module)
        if cls is not None:
            self.params_lst.append(cls.Params.from_torch_module(module, *args))
        return super().call_module(target, args, kwargs)


def scan_modules(model: torch.nn.Module, *args) -> List:
    """Run the model once on ``args`` and return the Params of every module that
    :func:`transform` would replace, in execution order."""
    interp = _ScanInterpreter(fx.symbolic_trace(model))
    interp.run(*args)
    return interp.params_lst
