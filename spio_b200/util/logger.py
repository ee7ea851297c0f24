"""Console logging controlled by SPIO_LOGGER (0 quiet, 1 info, 2 verbose), as in the
reference (spio/util/logger.py:7-18)."""

import os

_level = int(os.environ.get("SPIO_LOGGER", "0") or 0)
logger_enabled = _level > 0
logger_verbose = _level > 1


def log(message: str, verbose: bool = False) -> None:
    if logger_verbose or (logger_enabled and not verbose):
        print(f"spio: {message}", flush=True)
