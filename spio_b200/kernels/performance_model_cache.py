"""Chooses the tile configuration of a kernel for a layer shape.

The reference downloads per-device XGBoost models and returns the configuration with the
lowest predicted latency (spio/kernels/performance_model_cache.py:85-240, 432-479).  Here
the choice comes, in order, from

1. a tuning table: exact (kernel, params) entries measured on a B200 by
   ``spio_b200.kernels.autotune`` and stored as JSON (shipped in
   ``spio_b200/kernels/perf_models/`` and, for new measurements, in the user cache dir);
2. a learned model for the kernel (gradient-boosted trees stored as JSON, evaluated in
   pure Python), when one is shipped for this architecture;
3. the launch planner's own defaults (an all-zero configuration).

Architectures other than sm_100a raise NotImplementedError, as the reference does for
architectures it has no model for.
"""

from __future__ import annotations

import json
import os
from dataclasses import fields
from pathlib import Path
from typing import Any, Dict, Optional

from ..cuda.driver import get_device_attributes
from ..util.logger import log
from ..util.tensor_format import get_device_ordinal

MODEL_DIR = Path(__file__).resolve().parent / "perf_models"
SUPPORTED_ARCH = ("sm_100a",)


def user_cache_dir() -> Path:
    root = os.environ.get("SPIO_CACHE_DIR") or os.path.join(
        os.environ.get("XDG_CACHE_HOME", os.path.expanduser("~/.cache")), "spio_b200")
    return Path(root)


def params_features(params, skip=()) -> Dict[str, float]:
    """Flat numeric features of a params dataclass (padding split into its two values)."""
    out: Dict[str, float] = {}
    for f in fields(params):
        if f.name in skip:
            continue
        v = getattr(params, f.name)
        if f.name == "padding":
            out["padding_h"], out["padding_w"] = float(params.padding_h), float(params.padding_w)
        else:
            out[f.name] = float(v)
    return out


class PerformanceModelCache:
    def __init__(self):
        self._tables: Dict[str, Dict[str, Dict[str, int]]] = {}
        self._models: Dict[str, Any] = {}

    # ------------------------------------------------------------ tuning tables
    def _table(self, kernel_name: str, arch: str) -> Dict[str, Dict[str, int]]:
        key = f"{kernel_name}__{arch}"
        if key not in self._tables:
            table: Dict[str, Dict[str, int]] = {}
            for directory in (MODEL_DIR, user_cache_dir()):
                path = directory / f"tuned__{key}.json"
                if path.exists():
                    table.update(json.loads(path.read_text()))
            self._tables[key] = table
        return self._tables[key]

    def record(self, kernel_name: str, arch: str, params, config, directory: Optional[Path] = None) -> Path:
        """Add a measured best configuration to the table kept in ``directory``."""
        directory = Path(directory) if directory is not None else user_cache_dir()
        directory.mkdir(parents=True, exist_ok=True)
        path = directory / f"tuned__{kernel_name}__{arch}.json"
        table = json.loads(path.read_text()) if path.exists() else {}
        table[params.encode()] = config.as_tune()
        path.write_text(json.dumps(table, indent=1, sort_keys=True) + "\n")
        self._tables.pop(f"{kernel_name}__{arch}", None)
        return path

    # ------------------------------------------------------------ learned models
    def _model(self, kernel_name: str, arch: str):
        key = f"{kernel_name}__{arch}"
        if key not in self._models:
            path = MODEL_DIR / f"model__{key}.json"
            model = None
            if path.exists():
                from .gbt_model import GbtModel

                model = GbtModel.from_json(json.loads(path.read_text()))
                log(f"loaded performance model {path.name}", verbose=True)
            self._models[key] = model
        return self._models[key]

    # ------------------------------------------------------------ the choice
    def predict_best_kernel(self, kernel_factory, params, device, **kernel_kwargs):
        ordinal = get_device_ordinal(device)
        attr = get_device_attributes(ordinal)
        arch = attr.arch
        if arch not in SUPPORTED_ARCH:
            raise NotImplementedError(f"No performance model for device {attr.name} ({arch}); "
                                      f"supported: {SUPPORTED_ARCH}")
        kernel_name = kernel_factory.get_kernel_name(**kernel_kwargs)
        entry = self._table(kernel_name, arch).get(params.encode())
        if entry is not None:
            return kernel_factory.fixup_config(params, kernel_factory.config_cls(**entry), attr, **kernel_kwargs)
        model = self._model(kernel_name, arch)
        base = params_features(params, kernel_factory.per_model_skip_params)
        # the model is trusted only for filter sizes and image extents it was trained on
        if model is not None and model.covers(base, ("r", "s", "h", "w", "c")):
            configs = list(kernel_factory.configs(params, attr, **kernel_kwargs))
            if configs:
                rows = [dict(base, **{k: float(v) for k, v in c.as_tune().items()}) for c in configs]
                pred = model.predict(rows)
                return configs[min(range(len(configs)), key=pred.__getitem__)]
        return kernel_factory.config_cls()
