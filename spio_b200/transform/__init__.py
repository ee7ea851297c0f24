"""Model transformation (the names the reference exports from spio.transform)."""

from ._transform import transform, scan_modules
