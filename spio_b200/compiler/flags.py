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


class _ProcessFlag:
    """A process-wide switch with the get / set / reset methods of a ContextVar.  The choice
    between built-in and just-in-time kernels must also hold on autograd's worker threads,
    which do not inherit the context of the thread that called backward()."""

    def __init__(self, value: bool):
        self._value = value

    def get(self) -> bool:
        return self._value

    def set(self, value: bool) -> bool:
        old, self._value = self._value, bool(value)
        return old

    def reset(self, token: bool) -> None:
        self._value = token


jit = _ProcessFlag(env_var_is_true("SPIO_JIT"))
