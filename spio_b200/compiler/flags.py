"""Compiler settings taken from the environment (reference: spio/compiler/flags.py:7-22).

SPIO_LINEINFO / SPIO_DEBUG add -lineinfo / -G, SPIO_WORKERS sets the number of parallel
compilations, SPIO_JIT=1 makes every kernel compile just in time instead of using the
variants built into the library.  Listing machine code (the reference's SPIO_DISASM and
SPIO_COUNT_INSTRUCTIONS) is not offered.
"""

import os
from contextvars import ContextVar


def env_var_is_true(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() in ("1", "true", "yes", "on")


DEFAULT_WORKERS = 4

workers = max(1, int(os.environ.get("SPIO_WORKERS", str(DEFAULT_WORKERS))))
lineinfo = ContextVar("lineinfo", default=env_var_is_true("SPIO_LINEINFO"))
debug = ContextVar("debug", default=env_var_is_true("SPIO_DEBUG"))
jit = ContextVar("jit", default=env_var_is_true("SPIO_JIT"))
