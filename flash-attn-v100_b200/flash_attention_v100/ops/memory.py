"""Workspace sizing for the attention kernels.

Counterpart of the reference's ops/memory.py workspace functions
(allocate_attention_workspace_enhanced :653-760, estimate_peak_memory_usage_enhanced
:786-896).  The reference's tensor pool, background thread and leak detector
(:91-649) are not rebuilt: PyTorch's caching allocator already recycles blocks.
"""
from __future__ import annotations

import ctypes
from typing import Dict

import torch

from ..kernels import _cabi
from ..kernels.tile_table import dtype_enum


def _sizes_params(batch_size, seq_len_q, seq_len_k, num_heads, head_dim, dtype, num_heads_kv=None):
    p = _cabi.Params()
    p.struct_bytes = ctypes.sizeof(_cabi.Params)
    p.B, p.Nq, p.Nk, p.H, p.D = batch_size, seq_len_q, seq_len_k, num_heads, head_dim
    p.Hkv = num_heads if num_heads_kv is None else num_heads_kv
    p.dtype = dtype_enum(dtype)
    p.scale = 1.0          # any valid scale: the size does not depend on it, kernel selection checks it
    return p


def backward_workspace_bytes(batch_size: int, seq_len_q: int, seq_len_k: int, num_heads: int,
                             head_dim: int, dtype: torch.dtype, num_heads_kv: int = None) -> int:
    """Bytes of scratch fa_b200_bwd needs: delta (B,H,Nq) fp32 plus, for the
    tensor-core kernels, an fp32 dQ accumulator."""
    p = _sizes_params(batch_size, seq_len_q, seq_len_k, num_heads, head_dim, dtype, num_heads_kv)
    return int(_cabi.load().fa_b200_bwd_workspace_bytes(ctypes.byref(p)))


def dropout_bits_bytes(batch_size: int, seq_len_q: int, seq_len_k: int, num_heads: int, head_dim: int,
                       dtype: torch.dtype, dropout_p: float, num_heads_kv: int = None) -> int:
    """Bytes of the buffer that holds a call's dropout keep bits (two bits of storage per score: one per
    orientation), or 0 where the kernels draw their bits themselves (no dropout, CUDA-core kernels)."""
    p = _sizes_params(batch_size, seq_len_q, seq_len_k, num_heads, head_dim, dtype, num_heads_kv)
    p.dropout_p = float(dropout_p)
    return int(_cabi.load().fa_b200_dropout_bits_bytes(ctypes.byref(p)))


def allocate_attention_workspace(batch_size: int, seq_len_q: int, seq_len_k: int, num_heads: int,
                                 head_dim: int, dtype: torch.dtype, device: torch.device,
                                 include_backward: bool = True, enable_multi_gpu: bool = False,
                                 optimization_level: int = 1) -> Dict[str, torch.Tensor]:
    """Same buffer names and shapes as the reference (ops/memory.py:693-730):
    output, lse, grad_q/k/v; the reference's separate `delta` and `max_vals`
    buffers are folded into one `workspace` byte buffer sized by the library."""
    ws = {
        "output": torch.empty(batch_size, seq_len_q, num_heads, head_dim, dtype=dtype, device=device),
        "lse": torch.empty(batch_size, num_heads, seq_len_q, dtype=torch.float32, device=device),
    }
    if include_backward:
        ws["grad_q"] = torch.empty(batch_size, seq_len_q, num_heads, head_dim, dtype=dtype, device=device)
        ws["grad_k"] = torch.empty(batch_size, seq_len_k, num_heads, head_dim, dtype=dtype, device=device)
        ws["grad_v"] = torch.empty(batch_size, seq_len_k, num_heads, head_dim, dtype=dtype, device=device)
        n = backward_workspace_bytes(batch_size, seq_len_q, seq_len_k, num_heads, head_dim, dtype)
        ws["workspace"] = torch.empty(n, dtype=torch.uint8, device=device)
    return ws


def free_attention_workspace(workspace: Dict[str, torch.Tensor], defer_cleanup: bool = True) -> None:
    """Drop the references; the caching allocator keeps the blocks for reuse."""
    workspace.clear()


def estimate_peak_memory_usage(batch_size: int, seq_len_q: int, seq_len_k: int, num_heads: int,
                               head_dim: int, dtype: torch.dtype, include_gradients: bool = True,
                               dropout_p: float = 0.0, **_ignored) -> Dict[str, float]:
    """Bytes the op holds at its peak, in the reference's result keys
    (ops/memory.py:786-896: *_mb entries and total_memory_mb).  O(N) in the
    sequence length: no (N x N) score tensor is ever materialised; with dropout on
    the tensor-core kernels the call's keep bits are (Nq x Nk / 4 bytes per head)."""
    es = torch.empty((), dtype=dtype).element_size()
    t_q = batch_size * seq_len_q * num_heads * head_dim * es
    t_k = batch_size * seq_len_k * num_heads * head_dim * es
    lse = batch_size * num_heads * seq_len_q * 4
    fwd = t_q * 2 + t_k * 2 + lse                     # q, o, k, v, lse
    bwd = 0
    if include_gradients:
        bwd = t_q * 2 + t_k * 2                        # dO, dQ, dK, dV
        bwd += backward_workspace_bytes(batch_size, seq_len_q, seq_len_k, num_heads, head_dim, dtype)
    bits = dropout_bits_bytes(batch_size, seq_len_q, seq_len_k, num_heads, head_dim, dtype, dropout_p) \
        if dropout_p > 0.0 else 0
    if not include_gradients:
        bits //= 2                                     # a forward alone keeps one orientation
    mb = 1.0 / (1024 ** 2)
    return {"input_memory_mb": (t_q + 2 * t_k) * mb, "output_memory_mb": (t_q + lse) * mb,
            "gradient_memory_mb": bwd * mb, "dropout_bits_memory_mb": bits * mb,
            "total_memory_mb": (fwd + bwd + bits) * mb}


def get_memory_statistics(device=None) -> Dict[str, float]:
    """Allocator statistics (reference ops/memory.py:911-960 reports pool stats)."""
    if not torch.cuda.is_available():
        return {"allocated_mb": 0.0, "reserved_mb": 0.0, "peak_allocated_mb": 0.0}
    mb = 1.0 / (1024 ** 2)
    return {"allocated_mb": torch.cuda.memory_allocated(device) * mb,
            "reserved_mb": torch.cuda.memory_reserved(device) * mb,
            "peak_allocated_mb": torch.cuda.max_memory_allocated(device) * mb}


__all__ = ["backward_workspace_bytes", "allocate_attention_workspace", "free_attention_workspace",
           "estimate_peak_memory_usage", "get_memory_statistics"]
