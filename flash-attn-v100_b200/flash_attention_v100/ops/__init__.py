"""Operations package: the autograd op and workspace sizing.

Re-exports the names of the reference's ops/__init__.py (:8-41) that exist
here; the reference's MemoryManager pool is not rebuilt (PyTorch's caching
allocator already recycles blocks).
"""
from .attention import (
    FlashAttentionV100Function,
    flash_attention_forward,
    flash_attention_backward,
    compare_with_pytorch_attention,
    set_dropout_seed,
    kernel_variant,
)
from .memory import (
    allocate_attention_workspace,
    free_attention_workspace,
    estimate_peak_memory_usage,
    get_memory_statistics,
    backward_workspace_bytes,
)

from .host_pipeline import HostAttentionStep, chunk_bounds, plan_chunks
from .sequence_parallel import (
    flash_attention_v100_sequence_parallel,
    ring_schedule,
    zigzag_split,
    zigzag_merge,
)

__version__ = "0.1.0"

__all__ = [
    "FlashAttentionV100Function", "flash_attention_forward", "flash_attention_backward",
    "compare_with_pytorch_attention", "set_dropout_seed", "kernel_variant",
    "allocate_attention_workspace", "free_attention_workspace", "estimate_peak_memory_usage",
    "get_memory_statistics", "backward_workspace_bytes",
    "HostAttentionStep", "chunk_bounds", "plan_chunks",
    "flash_attention_v100_sequence_parallel", "ring_schedule", "zigzag_split", "zigzag_merge",
]
