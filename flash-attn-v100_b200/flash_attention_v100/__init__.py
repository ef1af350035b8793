"""flash_attention_v100 — exact attention forward/backward for NVIDIA B200.

Drop-in for the hot path of mini-kio/flash-attn-v100: the same import name and
public names (reference __init__.py:100-120, interface.py:663-673), the same
(B, N, H, D) tensor layout, hand-written sm_100a CUDA kernels underneath
instead of Triton.  There is no CPU or PyTorch fallback: the shared library
must be built (csrc/build.py) and a CUDA device must be present to compute.
"""
import torch

from .config import SUPPORTED_DTYPES, MIN_CUDA_VERSION, B200_COMPUTE_CAPABILITY, get_enhanced_config
from .interface import (
    flash_attention_v100,
    flash_attention_v100_causal,
    flash_attention_v100_with_dropout,
    flash_attention_v100_multi_gpu,
    FlashAttentionV100Manager,
    get_flash_attention_manager,
    flash_attention_performance_mode,
    flash_attention_memory_mode,
    plan_shards,
)
from .ops.attention import (
    FlashAttentionV100Function,
    flash_attention_forward,
    flash_attention_backward,
    compare_with_pytorch_attention,
    set_dropout_seed,
    kernel_variant,
)
from .ops.host_pipeline import HostAttentionStep
from .modules import EnhancedMultiHeadAttention
from .ops.sequence_parallel import flash_attention_v100_sequence_parallel

__version__ = "0.1.0"
__author__ = "flash_attention_v100 B200 build"


def _check_environment() -> bool:
    """Reference __init__.py:63-98 checks CUDA >= 11.0 and CC >= 7.0; the
    kernels here are sm_100a only."""
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is not available. flash_attention_v100 requires a CUDA device.")
    cap = torch.cuda.get_device_capability()
    if cap[0] != B200_COMPUTE_CAPABILITY[0]:
        raise RuntimeError(f"GPU compute capability {cap} is not supported: the kernels are built for "
                           f"sm_100a (compute capability {B200_COMPUTE_CAPABILITY}).")
    return True


try:
    _check_environment()
    _ENVIRONMENT_OK = True
except RuntimeError:
    # importable without a GPU (tile lookups, shard planning, validation); any
    # attempt to compute raises from the CUDA runtime
    _ENVIRONMENT_OK = False

__all__ = [
    "flash_attention_v100", "FlashAttentionV100Function", "SUPPORTED_DTYPES", "_ENVIRONMENT_OK",
    "__version__", "flash_attention_forward", "flash_attention_backward",
    "compare_with_pytorch_attention", "flash_attention_v100_causal",
    "flash_attention_v100_with_dropout", "flash_attention_v100_multi_gpu",
    "FlashAttentionV100Manager", "get_flash_attention_manager", "flash_attention_performance_mode",
    "flash_attention_memory_mode", "get_enhanced_config", "plan_shards", "set_dropout_seed",
    "kernel_variant", "HostAttentionStep", "EnhancedMultiHeadAttention",
    "flash_attention_v100_sequence_parallel",
]
