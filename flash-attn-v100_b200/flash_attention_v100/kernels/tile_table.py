"""Static tile table: (head_dim, dtype, causal, pass) -> tile configuration.

Replaces the reference's run-time tuner (kernels/autotuning.py:118-1018,
never reached from its call path) and the seq-len buckets of
config.get_enhanced_config (config.py:288-348).  The table lives in the shared
library: fa_b200_tile_config reports the constants of csrc/tile_config.cuh, the
header the kernels themselves are compiled from, so what this module returns is
what runs.
"""
from __future__ import annotations

import functools

import torch

from . import _cabi

_DTYPE_ENUM = {torch.float16: _cabi.FA_B200_F16, torch.bfloat16: _cabi.FA_B200_BF16,
               torch.float32: _cabi.FA_B200_F32}


def dtype_enum(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_ENUM[dtype]
    except KeyError:
        raise ValueError(f"Unsupported dtype {dtype}. Supported types: "
                         + ", ".join(str(d) for d in _DTYPE_ENUM)) from None


@functools.lru_cache(maxsize=None)
def lookup(head_dim: int, dtype: torch.dtype = torch.bfloat16, causal: bool = False,
           backward: bool = False) -> dict:
    """Tile configuration as a dict with the reference's key names
    (BLOCK_M, BLOCK_N, BLOCK_K, NUM_STAGES, NUM_WARPS) plus the kernel family."""
    t = _cabi.Tile()
    rc = _cabi.load().fa_b200_tile_config(int(head_dim), dtype_enum(dtype), int(causal), int(backward), t)
    _cabi.raise_for_status(rc, "fa_b200_tile_config")
    return {
        "BLOCK_M": t.block_m, "BLOCK_N": t.block_n, "BLOCK_K": int(head_dim),
        "NUM_STAGES": t.kv_stages, "NUM_WARPS": t.num_warps,
        "Q_TILES_PER_CTA": t.q_tiles_per_cta, "VARIANT": _cabi.VARIANT_NAMES[t.variant],
        "W_STAGES": t.w_stages, "REGS_SOFTMAX": t.regs_softmax, "REGS_OTHER": t.regs_other,
        "ONE_KERNEL_BACKWARD": bool(t.one_kernel_backward),
    }
