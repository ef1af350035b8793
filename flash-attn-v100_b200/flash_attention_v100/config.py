"""Configuration constants and tile selection for the B200 build.

Keeps the names callers of the reference's config.py use (SUPPORTED_DTYPES,
get_enhanced_config and its dict keys, config.py:288-348) and replaces the
V100 numbers (config.py:21-45, 351-360) by B200 ones.
"""
from __future__ import annotations

import torch

SUPPORTED_DTYPES = {torch.float16, torch.bfloat16, torch.float32}   # reference __init__.py:26
MIN_CUDA_VERSION = (12, 8)            # first toolkit with sm_100a / tcgen05
B200_COMPUTE_CAPABILITY = (10, 0)

_STRATEGIES = ("speed", "memory", "balanced", "adaptive",
               "speed_focused", "memory_focused")


class B200MemoryHierarchy:
    """Counterpart of V100MemoryHierarchy (config.py:21-45)."""
    HBM_BYTES = 180 * 1000 ** 3
    L2_BYTES = 126 * 1024 ** 2
    SHARED_MEMORY_PER_CTA = 227 * 1024
    TMEM_COLUMNS = 512                 # 32-bit columns x 128 lanes per SM
    NUM_SMS = 148
    WARP_SIZE = 32


class MultiGPUConfig:
    """Counterpart of MultiGPUConfig (config.py:143-171): how the (batch x heads)
    grid is split over the GPUs of one box.  Attention over (b, h) needs no
    exchange, so the only strategies are independent shards."""
    STRATEGIES = ("head_parallel", "batch_parallel", "grid_parallel")
    MAX_GPUS = 8


class PerformanceConfig:
    """Counterpart of PerformanceConfig.TARGET_METRICS (config.py:351-360)."""
    TARGET_METRICS = {
        "peak_tflops": 2250.0,           # B200 dense bf16/fp16 tensor peak (nominal)
        "target_forward_fraction": 0.60,
        "target_backward_fraction": 0.45,
        "hbm_gbs": 7700.0,
    }


def get_enhanced_config(seq_len: int, head_dim: int, num_gpus: int = 1,
                        strategy: str = "balanced", dtype: torch.dtype = torch.bfloat16,
                        causal: bool = False) -> dict:
    """Tile configuration for a problem; same keys as the reference's
    get_enhanced_config (config.py:288-348): BLOCK_M, BLOCK_N, BLOCK_K,
    NUM_STAGES, NUM_WARPS and the ENABLE_* flags.

    The values come from the static per-(head_dim, dtype, causal) tile table,
    not from sequence-length buckets; `strategy` is accepted for source
    compatibility and never changes results.
    """
    from .kernels import tile_table
    if strategy not in _STRATEGIES:
        strategy = "balanced"           # reference: unknown strategy -> 'balanced' (config.py:317-318)
    cfg = dict(tile_table.lookup(int(head_dim), dtype, bool(causal), False))
    cfg["BLOCK_K"] = int(head_dim)      # reference config.py:338
    if num_gpus > 1:
        cfg["ENABLE_MULTI_GPU"] = True
        cfg["NUM_GPUS"] = int(num_gpus)
        cfg["PARALLELIZATION_STRATEGY"] = "head_parallel"   # reference config.py:331-335
    cfg.update({
        "ENABLE_WARP_SPECIALIZATION": cfg["VARIANT"] == "tcgen05",
        "ENABLE_DOUBLE_BUFFERING": True,
        "ENABLE_KERNEL_FUSION": True,
        "MEMORY_ACCESS_OPTIMIZATION": True,
        "STRATEGY": strategy,
    })
    return cfg


__all__ = ["SUPPORTED_DTYPES", "MIN_CUDA_VERSION", "B200_COMPUTE_CAPABILITY", "B200MemoryHierarchy",
           "MultiGPUConfig", "PerformanceConfig", "get_enhanced_config"]
