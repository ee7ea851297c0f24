"""spio_b200: B200-native (sm_100a) grouped conv2d with group width 8.

Importing the package touches neither CUDA nor the native library; both are loaded on
first use (the reference initialises the driver at import, spio/__init__.py:8-14).
"""

__version__ = "0.2.0"

supported_arch = ["sm_100a"]


def check_status() -> None:
    """Synchronise the current CUDA device and raise ``ValueError`` if a kernel recorded a bounded
    wait that gave up since the last check (the outputs of that launch are then incomplete).

    Every wait inside the kernels ends after two seconds of wall time instead of spinning for ever;
    the kernel then records the fact in a per-device status word and returns.  The operators do not
    read that word on their own (it would cost a device synchronisation per call); call this at a
    point that synchronises anyway, for instance once per optimizer step, or set ``SPIO_CHECK_STATUS=1``
    to have every backward pass of ``spio::conv2d_gw8`` check it.  The reference reports driver
    errors as ``ValueError`` the same way (spio/cuda/driver.pyx:118-123)."""
    from . import _clib

    code = _clib.device_status()
    if code != 0:
        what = {1: "a barrier wait inside a convolution kernel", 2: "the data-parallel exchange (a peer's data)"}
        raise ValueError(f"CUDA error: a bounded wait gave up: {what.get(code, 'status ' + str(code))}; "
                         "the results of that launch are incomplete")
