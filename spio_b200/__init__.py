"""spio_b200: B200-native (sm_100a) grouped conv2d with group width 8.

Importing the package touches neither CUDA nor the native library; both are loaded on
first use (the reference initialises the driver at import, spio/__init__.py:8-14).
"""

__version__ = "0.1.0"

supported_arch = ["sm_100a"]
