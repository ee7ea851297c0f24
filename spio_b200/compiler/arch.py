"""Architecture names for the compiler command line.

The reference maps a compute-capability tuple to ``sm_XY`` (spio/compiler/arch.py:6-10).
The kernels of this package use TMA and mbarrier features that NVRTC accepts only for the
architecture-specific target, so capability 9.0 and above get the ``a`` suffix.
"""

from typing import Tuple, Union


def sm_from_arch(arch: Union[Tuple[int, int], str, None]) -> Union[str, None]:
    if isinstance(arch, tuple):
        major, minor = arch
        return f"sm_{major}{minor}" + ("a" if major >= 9 else "")
    return arch
