"""Device access: attributes now, the driver-API module loader for JIT kernels in driver.py."""

from .driver import DeviceAttributes, get_device_attributes, B200_ATTRIBUTES
