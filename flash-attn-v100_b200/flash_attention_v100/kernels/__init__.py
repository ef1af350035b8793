"""Launch layer: ctypes binding of the sm_100a kernels and the static tile table.

Counterpart of the reference's kernels/ package (kernels/__init__.py:1-79),
whose Triton kernels and autotuner are replaced by libfa_b200.so.
"""
from . import _cabi, tile_table

__all__ = ["_cabi", "tile_table"]
