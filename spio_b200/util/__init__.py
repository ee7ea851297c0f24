"""Small helpers shared by the package (tolerances, layouts, logging, integer math)."""

from .close import assert_all_close, assert_all_close_with_acc_depth
from .logger import logger_enabled, logger_verbose, log
from .math import divup, next_relative_prime
from .tensor_format import check_channels_last, to_channels_last, get_device_ordinal
